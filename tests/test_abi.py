"""CPU-only checks of the C-ABI boundary: the library loads, exports every symbol the
header declares, and rejects bad requests on the host before touching a device."""

import ctypes as C
import re
from pathlib import Path

import pytest

from superl8_b200 import _lib

ROOT = Path(__file__).resolve().parent.parent
HEADER = ROOT / "include" / "superl8_b200.h"


def declared_symbols():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(sl8_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_all_exported_and_bound():
    lib = _lib.load()
    names = declared_symbols()
    assert len(names) >= 16
    for n in names:
        assert hasattr(lib, n), f"{n} declared in the header but not exported"
        assert n in _lib.SIGNATURES, f"{n} has no ctypes signature"
    assert lib.sl8_abi_version() == 1


def test_status_strings_carry_the_reference_key_words():
    assert "num_splits" in _lib.status_string(_lib.ERR_BAD_NUM_SPLITS)
    assert "float16 or bfloat16" in _lib.status_string(_lib.ERR_BAD_DTYPE)
    assert "head dim" in _lib.status_string(_lib.ERR_BAD_HEAD_DIM)
    assert _lib.status_string(0) == "ok"


def test_host_side_validation_needs_no_device():
    lib = _lib.load()
    p = _lib.DecodeParams(B=1, Hq=8, Hkv=2, N=128, D=96, num_splits=-1)
    assert lib.sl8_attn_int8_decode(C.byref(p), None, 0, None) == _lib.ERR_BAD_HEAD_DIM
    for ns in (0, 257, -2):
        p = _lib.DecodeParams(B=1, Hq=8, Hkv=2, N=128, D=128, num_splits=ns)
        assert lib.sl8_attn_int8_decode(C.byref(p), None, 0, None) == _lib.ERR_BAD_NUM_SPLITS
    p = _lib.DecodeParams(B=1, Hq=8, Hkv=3, N=128, D=128, num_splits=1)
    assert lib.sl8_attn_int8_decode(C.byref(p), None, 0, None) == _lib.ERR_BAD_SHAPE
    f = _lib.FwdParams(B=1, Hq=4, Hkv=2, M=64, N=64, D=96, v_dtype=0)
    assert lib.sl8_attn_int8_fwd(C.byref(f), None, 0, None) == _lib.ERR_BAD_HEAD_DIM
    f = _lib.FwdParams(B=1, Hq=4, Hkv=2, M=64, N=64, D=128, v_dtype=2)
    assert lib.sl8_attn_int8_fwd(C.byref(f), None, 0, None) == _lib.ERR_BAD_DTYPE
    f = _lib.FwdParams(B=1, Hq=4, Hkv=2, M=0, N=64, D=128, v_dtype=0)
    assert lib.sl8_attn_int8_fwd(C.byref(f), None, 0, None) == 0          # empty output is a no-op
    f = _lib.FwdParams(B=1, Hq=4, Hkv=2, M=64, N=64, D=128, v_dtype=0)
    assert lib.sl8_attn_int8_fwd(C.byref(f), None, 0, None) == _lib.ERR_NULL
    assert lib.sl8_quantize_i8_rowwise(None, 0, 0, 128, None, None, None) == 0
    assert lib.sl8_quantize_i8_rowwise(None, 0, 4, 128, None, None, None) == _lib.ERR_NULL
    assert lib.sl8_quantize_i8_rowwise(None, 7, 4, 128, C.c_void_p(16), C.c_void_p(16), None) == _lib.ERR_NULL
    # the one-call forward: head dims of the tensor-memory kernels only, one 16-bit dtype, pointers checked
    u = _lib.FusedFwdParams(B=1, Hq=4, Hkv=2, M=64, N=64, D=80, dtype=0, softmax_scale=0.1)
    assert lib.sl8_attn_int8_fwd_fused(C.byref(u), None, 0, None) == _lib.ERR_UNSUPPORTED
    u = _lib.FusedFwdParams(B=1, Hq=4, Hkv=2, M=64, N=64, D=128, dtype=2, softmax_scale=0.1)
    assert lib.sl8_attn_int8_fwd_fused(C.byref(u), None, 0, None) == _lib.ERR_BAD_DTYPE
    u = _lib.FusedFwdParams(B=1, Hq=4, Hkv=3, M=64, N=64, D=128, dtype=0, softmax_scale=0.1)
    assert lib.sl8_attn_int8_fwd_fused(C.byref(u), None, 0, None) == _lib.ERR_BAD_SHAPE
    u = _lib.FusedFwdParams(B=1, Hq=4, Hkv=2, M=0, N=64, D=128, dtype=0, softmax_scale=0.1)
    assert lib.sl8_attn_int8_fwd_fused(C.byref(u), None, 0, None) == 0        # empty output is a no-op
    u = _lib.FusedFwdParams(B=1, Hq=4, Hkv=2, M=64, N=64, D=128, dtype=0, softmax_scale=0.1)
    assert lib.sl8_attn_int8_fwd_fused(C.byref(u), None, 0, None) == _lib.ERR_NULL
    u = _lib.FusedFwdParams(q=16, k=16, v=16, out=16, B=1, Hq=4, Hkv=2, M=64, N=64, D=128, dtype=0, softmax_scale=0.1)
    assert lib.sl8_attn_int8_fwd_fused(C.byref(u), None, 0, None) == _lib.ERR_WORKSPACE
    need = lib.sl8_attn_int8_fwd_fused_workspace(C.byref(u))
    assert need >= 512 + 4 * 64 * 128 + 2 * 64 * 128 + 4 * (4 * 64 + 2 * 64) and need % 256 == 0
    # the backward: the tensor-memory passes serve D = 64 / 128 only; the device-side gate needs the tcgen05 backend
    b = _lib.BwdParams(B=1, Hq=2, Hkv=2, M=64, N=64, D=32, dtype=0, backend=_lib.SL8_BACKEND_TCGEN05,
                       q=16, k=16, v=16, o=16, dout=16, lse=16, dq=16, dk=16, dv=16)
    assert lib.sl8_attn_bwd(C.byref(b), C.c_void_p(16), 1 << 20, None) == _lib.ERR_UNSUPPORTED
    f = _lib.FwdParams(q=16, q_scale=16, k=16, k_scale=16, v=16, out=16, B=1, Hq=4, Hkv=2, M=64, N=64, D=128, v_dtype=0,
                       backend=_lib.SL8_BACKEND_MMA, gate_flag=16)
    assert lib.sl8_attn_int8_fwd(C.byref(f), C.c_void_p(16), 256, None) == _lib.ERR_UNSUPPORTED


def test_host_side_plans_and_argument_checks_need_no_device():
    """Chunk plan of the host-buffer entry, eligibility of the one-launch K prologue, workspace of the
    tensor-memory W8A8 route and the validation of the Hadamard entry: pure host code."""
    lib = _lib.load()
    cfg3 = dict(B=16, Hq=64, Hkv=8, M=8192, N=8192, D=128, dtype=0, causal=1, window_left=-1, ratio_threshold=12.0,
                softmax_scale=0.0884)
    # automatic plan: one chunk per batch element, the last element in quarters (short drain)
    assert lib.sl8_attn_int8_fwd_host_chunks(C.byref(_lib.HostFwdParams(**cfg3))) == 15 + 4
    for kvc, chunks in ((8, 16), (4, 32), (2, 64), (1, 128), (3, 64), (100, 16)):   # explicit width: uniform chunks (rounded down to a divisor of Hkv)
        assert lib.sl8_attn_int8_fwd_host_chunks(C.byref(_lib.HostFwdParams(kv_heads_per_chunk=kvc, **cfg3))) == chunks, kvc
    small = dict(cfg3, B=1, Hq=8, Hkv=2, M=1024, N=1024)                             # too small to cut: one chunk
    assert lib.sl8_attn_int8_fwd_host_chunks(C.byref(_lib.HostFwdParams(**small))) == 1
    assert lib.sl8_attn_int8_fwd_host_chunks(C.byref(_lib.HostFwdParams(**dict(cfg3, Hkv=3)))) == 0   # Hq % Hkv != 0
    ws3 = lib.sl8_attn_int8_fwd_host_workspace(C.byref(_lib.HostFwdParams(slots=3, **cfg3)))
    ws4 = lib.sl8_attn_int8_fwd_host_workspace(C.byref(_lib.HostFwdParams(slots=4, **cfg3)))
    one = 8 * 8 * 8192 * 128 * 2                                                      # Q bytes of a batch element
    assert ws3 % 256 == 0 and ws4 - ws3 == (ws3 - 256) // 3 and (ws3 - 256) // 3 >= 2 * one + 2 * one // 8
    h = _lib.HostFwdParams(q=16, k=16, v=16, out=16, **cfg3)
    assert lib.sl8_attn_int8_fwd_host(C.byref(h), None, 0, None) == _lib.ERR_WORKSPACE
    assert lib.sl8_attn_int8_fwd_host(C.byref(_lib.HostFwdParams(**cfg3)), None, 0, None) == _lib.ERR_NULL
    assert lib.sl8_attn_int8_fwd_host(C.byref(_lib.HostFwdParams(**dict(cfg3, D=80))), None, 0, None) == _lib.ERR_UNSUPPORTED
    assert lib.sl8_attn_int8_fwd_host(C.byref(_lib.HostFwdParams(**dict(cfg3, M=0))), None, 0, None) == 0
    # K prologue in one launch: 16-bit, the tensor-memory head dims, a slab short enough for the cluster's shared memory
    ok = lib.sl8_k_prologue_fused_ok
    assert ok(0, 128, 8192, 128) == 1 and ok(1, 8, 4096, 64) == 1 and ok(0, 1, 100, 256) == 1
    assert ok(2, 128, 8192, 128) == 0 and ok(0, 128, 8192, 80) == 0 and ok(0, 70000, 8192, 128) == 0 and ok(0, 0, 8, 128) == 0
    assert ok(0, 8, 1 << 20, 128) == 0            # 1024 chunks: their sums no longer fit the cluster's shared memory
    assert lib.sl8_k_prologue(None, 0, 0, 8, 128, None, 1, None, None, None, None, None) == 0     # empty
    assert lib.sl8_k_prologue(None, 0, 4, 8, 128, None, 1, None, None, None, None, None) == _lib.ERR_NULL
    assert lib.sl8_k_prologue(16, 2, 4, 8, 128, None, 1, 16, 16, 16, None, None) == _lib.ERR_UNSUPPORTED
    # W8A8 on the tensor-memory kernel: workspace = status area + V's codes as fp16
    w = _lib.W8A8Params(B=2, Hq=8, Hkv=2, M=300, N=500, D=128, causal=1, causal_diag=200, per_warp_quant=1)
    assert lib.sl8_attn_w8a8_fwd_tc_workspace(C.byref(w)) == 256 + 2 * 2 * 500 * 128 * 2
    assert lib.sl8_attn_w8a8_fwd_tc(C.byref(w), None, 0, None) == _lib.ERR_NULL
    for bad in (dict(D=32), dict(causal_diag=5), dict(N=0)):
        wb = _lib.W8A8Params(**{**dict(B=2, Hq=8, Hkv=2, M=300, N=500, D=128, causal=1, causal_diag=200, per_warp_quant=1), **bad})
        assert lib.sl8_attn_w8a8_fwd_tc(C.byref(wb), None, 0, None) == _lib.ERR_UNSUPPORTED, bad
    assert lib.sl8_attn_w8a8_fwd_tc(C.byref(_lib.W8A8Params(B=2, Hq=8, Hkv=2, M=0, N=500, D=128)), None, 0, None) == 0
    # Hadamard entry: 16-bit, power-of-two rows of 32 ... 1024 elements
    hq = lib.sl8_hadamard_quant_rows
    assert hq(None, 0, 0, 128, None, 1, 1.0, None, None, None, None) == 0
    assert hq(16, 2, 4, 128, None, 1, 1.0, 16, 16, None, None) == _lib.ERR_BAD_DTYPE
    for d in (96, 16, 2048):
        assert hq(16, 0, 4, d, None, 1, 1.0, 16, 16, None, None) == _lib.ERR_UNSUPPORTED, d
    assert hq(16, 0, 4, 128, None, 1, 1.0, None, None, None, None) == _lib.ERR_NULL            # nothing to write
    assert hq(16, 0, 4, 128, None, 1, 1.0, 16, None, None, None) == _lib.ERR_NULL              # codes without scales
    assert hq(24, 0, 4, 128, None, 1, 1.0, 16, 16, None, None) == _lib.ERR_MISALIGNED


def test_split_heuristic_properties():
    lib = _lib.load()
    assert lib.sl8_choose_n_splits(0, 8) == 1
    for n, bh in ((1024, 1024), (32768, 1024), (777, 8), (64000, 24), (100, 1), (2000, 16)):
        s = lib.sl8_choose_n_splits(n, bh)
        assert 1 <= s <= 256
        per = -(-n // s)
        assert per <= 2048 or s == 256
        assert s == 1 or per >= 128
    assert lib.sl8_choose_n_splits(32768, 1024) == 16
    p = _lib.DecodeParams(B=2, Hq=8, Hkv=2, N=4096, D=128, num_splits=4)
    assert lib.sl8_attn_int8_decode_workspace(C.byref(p)) == 256 + 4 * 16 * (128 + 2) * 4


def test_missing_library_raises_loudly(monkeypatch, tmp_path):
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", tmp_path / "nope.so")
    with pytest.raises(_lib.Sl8LibraryMissing, match="no CPU fallback"):
        _lib.load()


def test_python_layer_refuses_cpu_tensors():
    import torch
    import superl8_b200 as s8
    x = torch.randn(4, 128).half()
    with pytest.raises(RuntimeError, match="CUDA"):
        s8.quantize_i8_rowwise(x)
    with pytest.raises(RuntimeError, match="CUDA"):
        s8.quantize_int8_rowwise(x)
    with pytest.raises(RuntimeError, match="CUDA"):
        s8.attn_int8_fwd(x.view(1, 1, 4, 128), x.view(1, 1, 4, 128), x.view(1, 1, 4, 128))


STRUCTS = {
    "sl8_fwd_params": _lib.FwdParams, "sl8_fp16_fwd_params": _lib.Fp16FwdParams,
    "sl8_decode_params": _lib.DecodeParams, "sl8_w8a8_params": _lib.W8A8Params,
    "sl8_varlen_params": _lib.VarlenParams, "sl8_bwd_params": _lib.BwdParams,
    "sl8_fused_fwd_params": _lib.FusedFwdParams, "sl8_host_fwd_params": _lib.HostFwdParams,
}


def test_ctypes_structs_have_the_layout_the_c_compiler_gives_the_header(tmp_path):
    """Every parameter struct of the header, compiled as plain C, has the field order, offsets
    and size of its ctypes mirror (a silent mismatch would hand kernels shifted pointers)."""
    import shutil
    import subprocess
    gcc = shutil.which("gcc")
    if gcc is None:
        pytest.skip("no C compiler")
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    found = set(re.findall(r"typedef struct (sl8_[a-z0-9_]+)", text))
    assert found == set(STRUCTS), f"header structs {sorted(found)} vs ctypes mirrors {sorted(STRUCTS)}"
    lines = ['#include <stdio.h>', '#include <stddef.h>', f'#include "{HEADER}"', "int main(void) {"]
    for cname, cls in STRUCTS.items():
        lines.append(f'  printf("{cname} size %zu\\n", sizeof({cname}));')
        for fname, _ in cls._fields_:
            lines.append(f'  printf("{cname} {fname} %zu\\n", offsetof({cname}, {fname}));')
    lines += ["  return 0;", "}"]
    src = tmp_path / "layout.c"
    src.write_text("\n".join(lines))
    exe = tmp_path / "layout"
    subprocess.run([gcc, "-std=c99", "-Wall", "-Werror", str(src), "-o", str(exe)], check=True)
    out = subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout
    got = {(a, b): int(c) for a, b, c in (ln.split() for ln in out.splitlines())}
    for cname, cls in STRUCTS.items():
        assert got[(cname, "size")] == C.sizeof(cls), cname
        for fname, _ in cls._fields_:
            assert got[(cname, fname)] == getattr(cls, fname).offset, f"{cname}.{fname}"
        # and the header has no field the mirror lacks
        body = re.search(r"typedef struct %s \{(.*?)\} %s;" % (cname, cname), text, flags=re.S).group(1)
        n_fields = sum(len(decl.split(",")) for decl in body.split(";") if decl.strip())
        assert n_fields == len(cls._fields_), f"{cname}: {n_fields} fields in the header"


@pytest.mark.gpu
def test_bounded_wait_expires_with_a_status_and_leaves_the_context_usable(device):
    # The one allowed way to see SL8_ERR_DEVICE_TIMEOUT: a one-block self-test waits 1 ms on a barrier
    # nothing arrives at, with the same wait routine every kernel uses, and returns normally.
    import torch

    lib = _lib.load()
    torch.cuda.set_device(device)
    ws = torch.zeros(64, dtype=torch.int32, device=device)
    assert lib.sl8_wait_timeout_selftest(C.c_void_p(ws.data_ptr()), 256, 1_000_000, None) == 0
    torch.cuda.synchronize()
    assert int(ws[1].item()) == 2                                    # the wait gave up
    assert lib.sl8_read_device_status(C.c_void_p(ws.data_ptr()), None) == _lib.ERR_DEVICE_TIMEOUT
    assert lib.sl8_read_device_status(C.c_void_p(ws.data_ptr()), None) == 0   # reading cleared it
    # limits outside (0, 0.1 s] are refused on the host
    assert lib.sl8_wait_timeout_selftest(C.c_void_p(ws.data_ptr()), 256, 0, None) == _lib.ERR_BAD_SHAPE
    assert lib.sl8_wait_timeout_selftest(C.c_void_p(ws.data_ptr()), 256, 10**10, None) == _lib.ERR_BAD_SHAPE
    # the context is fine: a real kernel runs and is right
    x = torch.randn(64, 128, device=device, dtype=torch.float16)
    from superl8_b200 import _C
    q, s = _C.quantize_i8_rowwise(x)
    assert torch.equal(s, x.float().abs().amax(-1) * torch.tensor(1.0 / 127.0, dtype=torch.float32, device=device))
    assert _C.device_status() == 0
