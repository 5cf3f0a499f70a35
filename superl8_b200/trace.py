"""Reader for the clock-stamp traces of the tensor-memory kernels (a measuring aid, not a product path).

Recipe::

    python -m superl8_b200.build --trace [-DSL8_TRACE_BASE=n] [-DSL8_TRACE_STRIDE=m]
    SUPERL8_B200_LIB=superl8_b200/libsuperl8_b200_trace.so python - <<'EOF'
    import torch, superl8_b200 as s8
    from superl8_b200 import _C, trace
    _C.use_binding("ctypes")                      # the compiled binding links the shipped library
    ...                                           # one launch of the kernel under study
    torch.cuda.synchronize()
    t = trace.read("fwd")                         # int64 [8 blocks, 8192 slots], 0 = never stamped
    print(trace.periods(t[0], first_slot=0, stride=8, tiles=64))
    EOF

The trace build stamps ``clock64()`` where the kernel sources say ``TR(slot)`` for the eight blocks
whose linear index is SL8_TRACE_BASE + k * SL8_TRACE_STRIDE (csrc/sl8_common.cuh).  Slot layout of
``fwd_tc_kernel`` (csrc/fwd_tcgen05.cu): softmax warp 0 stamps 8 j + {0: before the S_FULL wait, 1: after
it, 2: logits in registers, 3: sweep done, 4: P complete, 5: arrived} for key tile j; the issuing warp
stamps 4096 + 8 j + {0: before the P_FULL wait, 1: after it, 2: P.V queued, 3: next Q.K^T queued};
8185-8187 bracket the epilogue, 8188/8189 the set-up, 8191 holds the SM id.  ``fwd_tc2_kernel`` and the
backward passes document theirs beside their ``TR`` calls."""

from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib

BLOCKS, SLOTS = 8, 8192
_READERS = {"fwd": "sl8_dbg_read_trace", "fwd_2q": "sl8_dbg_read_trace2", "bwd": "sl8_dbg_read_trace_bwd"}


def read(kernel: str = "fwd") -> np.ndarray:
    """Copies the stamps of the last launch back: int64 [8, 8192].  Raises when the loaded library is
    not a trace build."""
    lib = _lib.load()
    try:
        fn = getattr(lib, _READERS[kernel])
    except AttributeError as e:
        raise RuntimeError("superl8_b200.trace: the loaded library is not a trace build "
                           "(python -m superl8_b200.build --trace, then SUPERL8_B200_LIB=...)") from e
    fn.restype = C.c_int
    buf = (C.c_longlong * (BLOCKS * SLOTS))()
    rc = fn(buf, BLOCKS * SLOTS)
    if rc != 0:
        raise RuntimeError(f"superl8_b200.trace: reading the trace failed (cudaError {rc})")
    return np.frombuffer(buf, dtype=np.int64).reshape(BLOCKS, SLOTS).copy()


def periods(block: np.ndarray, first_slot: int, stride: int, tiles: int, skip: int = 4) -> dict:
    """Mean cycles between consecutive stamps of one per-tile slot (steady state: ``skip`` tiles
    dropped at both ends) and the mean length of every segment inside a tile."""
    s = block[first_slot:first_slot + stride * tiles].reshape(tiles, stride)
    valid = [j for j in range(tiles) if s[j, 0] > 0]
    if len(valid) < 2 * skip + 2:
        return {"tiles": len(valid)}
    j0, j1 = valid[skip], valid[-skip - 1]
    out = {"tiles": len(valid), "period": float(s[j1, 0] - s[j0, 0]) / (j1 - j0)}
    for c in range(1, stride):
        if (s[j0:j1, c] > 0).all() and (s[j0:j1, c - 1] > 0).all():
            out[f"seg{c - 1}->{c}"] = float(np.mean(s[j0:j1, c] - s[j0:j1, c - 1]))
    return out
