"""Python entry points with the reference's signatures (reference superl8/ops.py:70-267)."""

from __future__ import annotations

import math
import threading

import torch

from . import _C, _lib
from .quant import (_capturing, k_mean, k_prologue, q_outlier_flag, quantize_q, quantize_qk, smooth_quantize_k,
                    varlen_smooth_quantize_k)

# The outcome of the accuracy gate of the most recent attn_int8_fwd call, kept per (device, stream):
# calls on different streams or threads do not see each other's decision.  Read it with
# last_gate(device) -- or through the module attributes ``last_gate_decision`` / ``last_gate_flag``,
# which answer for the current stream of the current device.
_gate_lock = threading.Lock()
_gate_state: dict = {}


def _gate_key(device=None):
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    idx = device.index if device.index is not None else torch.cuda.current_device()
    return (idx, torch.cuda.current_stream(device).cuda_stream)


def _set_gate(device, decision, flag=None):
    with _gate_lock:
        _gate_state[_gate_key(device)] = (decision, flag)


def last_gate(device=None):
    """(decision, flag) of the most recent attn_int8_fwd call on the current stream of ``device``:
    decision is True (demoted to the full-precision kernel), False (int8 kernel), or None (gate off,
    skipped under capture, or decided on the device -- then ``flag`` is the int32 [1] device flag)."""
    if not torch.cuda.is_available():
        return (None, None)
    with _gate_lock:
        return _gate_state.get(_gate_key(device), (None, None))


def __getattr__(name):
    if name == "last_gate_decision":
        return last_gate()[0]
    if name == "last_gate_flag":
        return last_gate()[1]
    raise AttributeError(name)


def _demote(q, k, v, causal, s, window_left, seqlens_q, seqlens_k):
    """The gate's demotion target: the full-precision kernel (reference superl8/ops.py:120-130)."""
    if not (v.dtype == q.dtype and k.dtype == q.dtype):
        q, k = q.to(v.dtype), k.to(v.dtype)
    return _C.attn_fp16_fwd(q, k, v, causal, s, window_left, None, seqlens_q=seqlens_q, seqlens_k=seqlens_k)


def attn_int8_fwd(q, k, v, *, causal: bool = False, scale: float | None = None, int8_pv: bool = False,
                  rotate: bool = False, window_left: int = -1, per_warp_quant: bool = True,
                  internal_accuracy_gate: bool = True, seqlens_q=None, seqlens_k=None,
                  backend: int = _lib.SL8_BACKEND_AUTO, expect_demotion: bool | None = None):
    """INT8-QK FlashAttention-2 forward; q, k, v fp16/bf16 [B, H, S, D]; output in v's dtype.

    Same contract as the reference entry (superl8/ops.py:70-175): per-row int8 Q and
    smoothed K with exp2-ready folded scales, fp32 softmax, 16-bit P.V, bottom-right
    aligned causal mask, optional left window.  The accuracy gate (any Q row with
    max|q|/median|q| > 12) is asked FIRST, on the original q, and demotes the whole call to the
    full-precision kernel -- also when ``int8_pv=True``, exactly as the reference orders it
    (superl8/ops.py:121 before :152).  ``int8_pv=True`` otherwise takes the full-W8A8 route (V
    per-channel int8, P re-quantised per tile; ``per_warp_quant`` picks the finer per-32-key P
    scale; fp16 output; no window).  The gate costs one 4-byte device->host read and is skipped
    during CUDA-graph capture like the reference's.  By default its statistic is gathered inside
    the Q quantisation pass; when the previous call on this stream was demoted (or
    ``expect_demotion=True``) a read-only pass asks the gate before anything is quantised, so a
    stream of demoted calls does not quantise a Q nobody uses.  Both orders give the same result.
    ``internal_accuracy_gate="device"`` (not in the reference) keeps the decision on the GPU: the
    int8 kernel and the full-precision kernel are both launched on the same output and each
    reads the flag the Q pass raised, the one whose turn it is not exits at once.  No host
    read-back, so nothing stalls the stream and the gated call can be captured in a CUDA graph
    (the reference skips its gate under capture); ``last_gate()`` then returns (None, flag).
    Head dims 64/128/256 with one dtype for q, k, v; other cases take the host-side gate.
    ``seqlens_q`` / ``seqlens_k`` (int32 [B], not in the reference) give per-sequence
    lengths for padded ragged batches; the padding of k and v must hold finite numbers (rows of the
    last tile past a sequence's length are loaded and multiplied by a P of exactly 0).  A negative ``scale`` is served by the warp-level
    backend (the tensor-memory kernel takes row maxima before scaling and wants scale >= 0).
    """
    s = (1.0 / math.sqrt(q.shape[-1])) if scale is None else scale
    dev = q.device
    if int8_pv:
        if seqlens_q is not None or seqlens_k is not None:
            raise ValueError("seqlens are only supported on the fp16-PV path (int8_pv=False)")
        use_gate = bool(internal_accuracy_gate) and not _capturing()
        if use_gate and bool(q_outlier_flag(q).item()):
            _set_gate(dev, True)
            return _demote(q, k, v, causal, s, window_left, None, None)
        if window_left >= 0:
            raise ValueError("window_left is only supported on the fp16-PV path (int8_pv=False)")
        from .quant import quantize_v_perchannel

        q_i8, q_scale, k_i8, k_scale, _ = quantize_qk(q, k, softmax_scale=s, rotate=rotate)
        v_i8, v_scale = quantize_v_perchannel(v)
        _set_gate(dev, False if use_gate else None)
        return _C.attn_w8a8_fwd(q_i8, q_scale.squeeze(-1).contiguous(), k_i8, k_scale.squeeze(-1).contiguous(), v_i8,
                                v_scale.squeeze(-2).contiguous(), causal,
                                causal_diag=(k.shape[-2] - q.shape[-2]) if causal else 0, per_warp_quant=per_warp_quant)
    if (internal_accuracy_gate == "device" and not rotate and q.shape[-1] in (64, 128, 256) and k.shape[-2] > 0
            and q.dtype == k.dtype == v.dtype and backend in (_lib.SL8_BACKEND_AUTO, _lib.SL8_BACKEND_TCGEN05)
            and s >= 0):
        # one library call queues the gate, the prologue and both candidate kernels
        out, flag = _C.attn_int8_fwd_fused(q, k, v, causal, s, window_left, seqlens_q=seqlens_q, seqlens_k=seqlens_k)
        _set_gate(dev, None, flag)
        return out
    internal_accuracy_gate = bool(internal_accuracy_gate)
    use_gate = internal_accuracy_gate and not _capturing()
    if (_C._compiled() and not rotate and seqlens_q is None and seqlens_k is None and backend == _lib.SL8_BACKEND_AUTO
            and q.is_cuda and q.dim() == 4 and q.dtype == k.dtype == v.dtype and q.dtype in (torch.float16, torch.bfloat16)):
        # the whole step in one call of the compiled extension (same kernels, same order, same gate read)
        ask_first = last_gate(dev)[0] if expect_demotion is None else expect_demotion
        out, demoted = _C._ext.attn_int8_prefill(q, k, v, bool(causal), float(s), int(window_left), use_gate,
                                                 bool(use_gate and ask_first))
        if out.numel():
            kp = _lib.k_prologue_launches(_C._DTYPE[k.dtype], k.shape[0] * k.shape[1], k.shape[2], k.shape[3])
            _lib.launches += 2 if demoted else (2 + kp + (1 if (use_gate and ask_first) else 0))
        _set_gate(dev, bool(demoted) if use_gate else None)
        return out
    if s < 0 and backend == _lib.SL8_BACKEND_AUTO:
        backend = _lib.SL8_BACKEND_MMA
    if rotate:
        if use_gate and bool(q_outlier_flag(q).item()):
            _set_gate(dev, True)
            return _demote(q, k, v, causal, s, window_left, seqlens_q, seqlens_k)
        q_i8, q_scale, k_i8, k_scale, _ = quantize_qk(q, k, softmax_scale=s, rotate=True, seqlens_k=seqlens_k)
    else:
        ask_first = last_gate(dev)[0] if expect_demotion is None else expect_demotion
        if use_gate and ask_first:
            # ask the gate first (one read of Q, as the reference orders it) instead of quantising a
            # Q that is probably not going to be used
            demote = bool(q_outlier_flag(q).item())
            if not demote:
                q_i8, q_scale, _ = quantize_q(q, s, want_gate=False)
        else:
            # gate statistic fused into the quantisation pass
            q_i8, q_scale, flag = quantize_q(q, s, want_gate=use_gate)
            demote = use_gate and bool(flag.item())
        if demote:
            _set_gate(dev, True)
            return _demote(q, k, v, causal, s, window_left, seqlens_q, seqlens_k)
        k_i8, k_scale, _, _ = k_prologue(k, seqlens_k)
    _set_gate(dev, False if use_gate else None)
    return _C.attn_int8_fwd(q_i8, q_scale.squeeze(-1).contiguous(), k_i8, k_scale.squeeze(-1).contiguous(),
                            v.contiguous(), causal, window_left, seqlens_q=seqlens_q, seqlens_k=seqlens_k,
                            backend=backend)


_aux_streams: dict = {}
_host_ws: dict = {}      # per device: the staging workspace of attn_int8_fwd_host, kept between calls


def _host_workspace(dev, nbytes: int) -> torch.Tensor:
    buf = _host_ws.get(dev.index)
    if buf is None or buf.numel() < nbytes:
        buf = torch.empty(nbytes, dtype=torch.uint8, device=dev)
        _host_ws[dev.index] = buf
    return buf


def attn_int8_fwd_host(q, k, v, out=None, *, chunk_batch: int | None = None, staging_slots: int = 3,
                       kv_heads_per_chunk: int = 0, gate_flags=None, **kw):
    """attn_int8_fwd for tensors that live in (pinned) host memory: q, k, v fp16/bf16 [B, H, S, D]
    on the CPU, result written to ``out`` (pinned CPU tensor, allocated when None) and returned.

    (batch, kv-head) units are independent, so the call is cut into chunks of whole units that
    travel through three streams -- host->device copies, prologue + attention kernels on the
    caller's current stream, device->host copies -- ``staging_slots`` deep, so that both copy
    directions and the kernels overlap.  The accuracy gate is evaluated per chunk (the same as
    calling the op on every chunk).  The caller's stream is ordered after the last device->host
    copy on return; the copies are asynchronous for pinned tensors and the host thread never waits.

    The pipeline runs inside the library (sl8_attn_int8_fwd_host: one call, gate decided on the
    device, staging slots kept per device between calls) for head dims 64/128/256, one 16-bit dtype,
    scale >= 0 and the keyword arguments causal / scale / window_left / internal_accuracy_gate
    (True, False or "device"; the host-side gate does not exist here).  ``gate_flags`` (pinned int32
    [chunks], optional) receives every chunk's gate flag.  Anything else (rotate, int8_pv, an
    explicit ``chunk_batch``) takes a Python loop over batch chunks with the same three streams."""
    if q.is_cuda or k.is_cuda or v.is_cuda:
        raise RuntimeError("superl8_b200 attn_int8_fwd_host: q, k, v must be host tensors (see attn_int8_fwd)")
    if not torch.cuda.is_available():
        raise RuntimeError("superl8_b200 attn_int8_fwd_host: needs a CUDA device")
    dev = torch.device("cuda", torch.cuda.current_device())
    B = q.shape[0]
    if out is None:
        out = torch.empty(q.shape, dtype=v.dtype).pin_memory()
    if B == 0 or q.numel() == 0:
        return out
    known = {"causal", "scale", "window_left", "internal_accuracy_gate"}
    s = kw.get("scale")
    s = (1.0 / math.sqrt(q.shape[-1])) if s is None else float(s)
    if (chunk_batch is None and set(kw) <= known and q.dim() == 4 and q.shape[-1] in (64, 128, 256)
            and q.dtype == k.dtype == v.dtype == out.dtype and q.dtype in (torch.float16, torch.bfloat16)
            and k.shape[-2] > 0 and s >= 0 and all(t.is_contiguous() for t in (q, k, v, out))):
        gate = kw.get("internal_accuracy_gate", True)
        p = _lib.HostFwdParams(
            q=q.data_ptr(), k=k.data_ptr(), v=v.data_ptr(), out=out.data_ptr(),
            gate_flags=None if gate_flags is None else gate_flags.data_ptr(),
            B=B, Hq=q.shape[1], Hkv=k.shape[1], M=q.shape[2], N=k.shape[2], D=q.shape[3], dtype=_C._DTYPE[q.dtype],
            causal=int(bool(kw.get("causal", False))), window_left=int(kw.get("window_left", -1)),
            ratio_threshold=12.0 if gate else 0.0, softmax_scale=s, kv_heads_per_chunk=int(kv_heads_per_chunk),
            slots=int(staging_slots))
        lib = _lib.load()
        n_chunks = int(lib.sl8_attn_int8_fwd_host_chunks(p))
        if gate_flags is not None and (gate_flags.dtype != torch.int32 or gate_flags.numel() < n_chunks or gate_flags.is_cuda):
            raise RuntimeError(f"superl8_b200 attn_int8_fwd_host: gate_flags must be a host int32 tensor of >= {n_chunks}")
        with torch.cuda.device(dev):
            nbytes = int(lib.sl8_attn_int8_fwd_host_workspace(p))
            ws = _host_workspace(dev, nbytes)
            rc = lib.sl8_attn_int8_fwd_host(p, ws.data_ptr(), ws.numel(), _C._stream(dev))
        kp = _lib.k_prologue_launches(_C._DTYPE[k.dtype], max(1, k.shape[1] * B // max(n_chunks, 1)), k.shape[2], k.shape[3])
        _lib.check(rc, "attn_int8_fwd_host", n_chunks * (2 + kp + (1 if gate else 0)))
        _set_gate(dev, None, None)
        return out
    nb = max(1, B // 16) if chunk_batch is None else max(1, int(chunk_batch))
    cur = torch.cuda.current_stream(dev)
    if dev.index not in _aux_streams:
        _aux_streams[dev.index] = (torch.cuda.Stream(dev), torch.cuda.Stream(dev))
    h2d, d2h = _aux_streams[dev.index]
    h2d.wait_stream(cur)
    ns = max(2, int(staging_slots))
    slots = [tuple(torch.empty((nb, *t.shape[1:]), dtype=t.dtype, device=dev) for t in (q, k, v)) for _ in range(ns)]
    freed = [None] * ns      # recorded on the compute stream when a slot's kernels are queued
    starts = list(range(0, B, nb))

    def upload(i):
        b0, b1, s = starts[i], min(B, starts[i] + nb), i % ns
        with torch.cuda.stream(h2d):
            if freed[s] is not None:
                h2d.wait_event(freed[s])
            for dst, src in zip(slots[s], (q, k, v)):
                dst[:b1 - b0].copy_(src[b0:b1], non_blocking=True)
            ev = torch.cuda.Event()
            ev.record(h2d)
        return ev

    arrived = upload(0)
    for i in range(len(starts)):
        b0, b1, s = starts[i], min(B, starts[i] + nb), i % ns
        nxt = upload(i + 1) if i + 1 < len(starts) else None     # queued before this chunk's gate sync
        cur.wait_event(arrived)
        o = attn_int8_fwd(*(t[:b1 - b0] for t in slots[s]), **kw)
        freed[s] = torch.cuda.Event()
        freed[s].record(cur)
        with torch.cuda.stream(d2h):
            d2h.wait_event(freed[s])
            out[b0:b1].copy_(o, non_blocking=True)
        o.record_stream(d2h)
        arrived = nxt
    for t3 in slots:
        for t in t3:
            t.record_stream(h2d)
    cur.wait_stream(d2h)
    return out


def attn_fp16_fwd(q, k, v, *, causal: bool = False, scale: float | None = None, mask=None, window_left: int = -1):
    """Full-precision forward (reference superl8/ops.py:178-227)."""
    return _C.attn_fp16_fwd(q.contiguous(), k.contiguous(), v.contiguous(), causal, scale, window_left, mask)


def attn_int8_varlen(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q: int, max_seqlen_k: int, *,
                     causal: bool = False, scale: float | None = None):
    """Packed variable-length int8 prefill (reference superl8/ops.py:318-364): q, k, v token-major
    [total_tokens, H, D] fp16, cu_seqlens int32 [batch + 1]; every sequence attends within itself,
    the causal diagonal is aligned to the sequence end; K is smoothed with the mean of the token's
    own sequence.  Returns [total_q, H, D] in v's dtype.  ``max_seqlen_k`` is accepted for
    signature compatibility (the reference uses it to detect equal-length batches on the host)."""
    softmax_scale = (1.0 / math.sqrt(q.shape[-1])) if scale is None else float(scale)
    q_i8, q_scale, _ = quantize_q(q, softmax_scale)
    k_i8, k_scale, _, _ = varlen_smooth_quantize_k(k, cu_seqlens_k)
    return _C.attn_int8_varlen(q_i8, q_scale.squeeze(-1).contiguous(), k_i8, k_scale.squeeze(-1).contiguous(),
                               v.contiguous(), cu_seqlens_q.contiguous(), cu_seqlens_k.contiguous(),
                               int(max_seqlen_q), causal)


def backward_cuda(q, k, v, out, lse, d_out, *, causal: bool = False, scale: float | None = None,
                  backend: int = _lib.SL8_BACKEND_AUTO):
    """Fused backward -> (dq, dk, dv) in the inputs' 16-bit dtype (reference superl8/ops.py:39-67).
    ``lse`` [B, H, M] fp32 (natural log) from the forward; when None it is produced by the
    full-precision forward kernel (the reference recomputes it with dense torch ops)."""
    sc = (1.0 / math.sqrt(q.shape[-1])) if scale is None else float(scale)
    if lse is None:
        _, lse = _C.attn_fp16_fwd(q, k, v, causal, sc, want_lse=True)
    return _C.attn_bwd(q.contiguous(), k.contiguous(), v.contiguous(), out.contiguous(), d_out.contiguous(),
                       lse.contiguous(), sc, causal, backend=backend)


def attn_int8_decode(q, k, v, *, scale: float | None = None, rotate: bool = False, num_splits: int | None = None):
    """Decode (M = 1) via split-KV from fp16 q, k, v; quantises Q and the whole K first,
    exactly like the reference entry (superl8/ops.py:230-267)."""
    assert q.shape[-2] == 1, f"decode expects M=1, got M={q.shape[-2]}"
    q_i8, q_scale, k_i8, k_scale, _ = quantize_qk(q, k, softmax_scale=scale, rotate=rotate)
    ns = -1 if num_splits is None else int(num_splits)
    return _C.attn_int8_decode(q_i8, q_scale.reshape(q.shape[0], q.shape[1], 1).contiguous(), k_i8,
                               k_scale.squeeze(-1).contiguous(), v.contiguous(), ns)


def attn_decode(q, k, v, **kw):
    """Alias of :func:`attn_int8_decode`."""
    return attn_int8_decode(q, k, v, **kw)


def attn_decode_int8_cache(q, k_i8, k_scale, v, *, scale: float | None = None, num_splits: int | None = None,
                           context_lens=None):
    """Decode against an ALREADY quantised K cache (int8 [B,Hkv,N,D] + fp32 [B,Hkv,N]) and an
    fp16 V cache: only the one-row Q is quantised per step.  This is the serving-time shape of
    the path (the reference quantises its query the same way for cached decode,
    superl8/ops.py:706-717); ``context_lens`` int32 [B] gives per-sequence lengths."""
    assert q.shape[-2] == 1, f"decode expects M=1, got M={q.shape[-2]}"
    s = (1.0 / math.sqrt(q.shape[-1])) if scale is None else scale
    q_i8, q_scale, _ = quantize_q(q, s)
    ns = -1 if num_splits is None else int(num_splits)
    return _C.attn_int8_decode(q_i8, q_scale.reshape(q.shape[0], q.shape[1], 1).contiguous(), k_i8, k_scale, v, ns,
                               context_lens=context_lens)


def quantize_kv_cache(k, v, *, v_quant: str = "per_channel", rotate: bool = False):
    """Quantise a K/V cache once for int8-KV decode (reference superl8/ops.py:541-589):
    K is smoothed (per-channel mean over its keys) and quantised per row; V is quantised per
    channel.  Returns (k_i8 [B,H,N,D], k_scale [B,H,N], v_i8 [B,H,N,D], v_scale [B,H,D]).
    ``v_quant="per_token"`` belongs to the reference's paged decode, which is not part of this
    library."""
    if v_quant not in ("per_channel", "per_token"):
        raise ValueError(f"v_quant must be 'per_channel' or 'per_token', got {v_quant!r}")
    if v_quant == "per_token":
        raise NotImplementedError("superl8_b200: per-token V scales are served by the reference's paged decode only")
    from .quant import _rotation_kernel_ok, hadamard_quantize_rows, quantize_v_perchannel, rotate_last

    mean = k_mean(k)
    if rotate and _rotation_kernel_ok(k):   # smoothing, rotation and quantisation of a row in one pass
        k_i8, k_scale, _ = hadamard_quantize_rows(k, mean=mean.reshape(*k.shape[:-2], k.shape[-1]))
        k_scale = k_scale.squeeze(-1)
    elif rotate:
        _, _, k_s = smooth_quantize_k(k, mean, want_smoothed=True)
        k_i8, k_scale = _C.quantize_i8_rowwise(rotate_last(k_s).reshape(-1, k.shape[-1]).contiguous())
        k_i8, k_scale = k_i8.reshape(k.shape), k_scale.reshape(*k.shape[:-1])
    else:
        k_i8, k_scale, _ = smooth_quantize_k(k, mean)
        k_scale = k_scale.squeeze(-1)
    v_i8, v_scale = quantize_v_perchannel(v)
    return k_i8.contiguous(), k_scale.contiguous(), v_i8, v_scale.squeeze(-2).contiguous()


def attn_decode_cached(q, k_i8, k_scale, v_i8, v_scale, *, scale: float | None = None, rotate: bool = False,
                       num_splits: int | None = None, context_lens=None):
    """Decode (M = 1) against a pre-quantised int8 K / int8 V cache from quantize_kv_cache
    (reference superl8/ops.py:671-727): only the query row is quantised per call.
    ``context_lens`` int32 [B] gives per-sequence lengths of a padded cache."""
    assert q.shape[-2] == 1, f"decode expects M=1, got M={q.shape[-2]}"
    if v_scale.shape[-1] == k_i8.shape[2] and v_scale.shape[-1] != k_i8.shape[3]:
        raise RuntimeError("attn_decode_cached received a per-token V scale [B,H,N]; this kernel takes "
                           "per-channel V scales [B,H,D]")
    s = (1.0 / math.sqrt(q.shape[-1])) if scale is None else scale
    if rotate:
        from .quant import LOG2E, _rotation_kernel_ok, hadamard_quantize_rows, rotate_last
        if _rotation_kernel_ok(q):
            q_i8, q_scale, _ = hadamard_quantize_rows(q, fold=s * LOG2E)
        else:
            q_i8, q_scale, _ = quantize_q(rotate_last(q), s)
    else:
        q_i8, q_scale, _ = quantize_q(q, s)
    ns = -1 if num_splits is None else int(num_splits)
    return _C.attn_int8_decode_kv8(q_i8, q_scale.reshape(q.shape[0], q.shape[1], 1).contiguous(), k_i8.contiguous(),
                                   k_scale.contiguous(), v_i8, v_scale, ns, context_lens=context_lens)


def quantize_i8_rowwise(x: torch.Tensor):
    """[M, K] -> (int8 [M, K], fp32 [M]) (reference superl8/ops.py:975-991; CUDA tensors only)."""
    return _C.quantize_i8_rowwise(x)
