"""Operator layer with the names and argument lists of the reference's compiled
module ``superl8._C`` (reference csrc/fni8_api.cpp:225-291), implemented over the
C ABI of ``libsuperl8_b200.so``.

Each function validates like the reference's ``TORCH_CHECK``s (same key words in
the messages), allocates outputs/workspaces with torch on the inputs' device and
launches on torch's current stream.  Nothing here computes on the CPU.
"""

from __future__ import annotations

import ctypes as C
import math

import torch

from . import _lib

# Two bindings serve the reference's six compiled operators (quantize_i8_rowwise, attn_int8_fwd,
# attn_int8_fwd_train, attn_fp16_fwd, attn_bwd, attn_int8_decode): the compiled torch extension
# ``_C_ext`` (csrc/torch_ext, built by ``python -m superl8_b200.build``) when it is present, and
# ctypes otherwise.  Both end in the same C-ABI calls.  Calls that use an argument the reference's
# operators do not have (seqlens, backend, out, gate_flag, context_lens) always take ctypes.
try:
    from . import _C_ext as _ext
except ImportError:          # not built: the ctypes binding serves everything
    _ext = None
BINDING = "compiled" if _ext is not None else "ctypes"


def use_binding(name: str) -> str:
    """Selects "compiled" or "ctypes" for the six reference operators; returns the previous choice."""
    global BINDING
    if name not in ("compiled", "ctypes"):
        raise ValueError(name)
    if name == "compiled" and _ext is None:
        raise RuntimeError("superl8_b200: the compiled extension _C_ext is not built (python -m superl8_b200.build)")
    prev, BINDING = BINDING, name
    return prev


def _compiled() -> bool:
    return BINDING == "compiled"


_DTYPE = {torch.float16: _lib.SL8_F16, torch.bfloat16: _lib.SL8_BF16, torch.float32: _lib.SL8_F32}
_status_ws: dict = {}
_decode_ws: dict = {}
_bwd_ws: dict = {}      # the last backward workspace per (device, stream): its status word is read by device_status


def _stream(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _ptr(t):
    return None if t is None else C.c_void_p(t.data_ptr())


def _status_buffer(device) -> torch.Tensor:
    key = (device.index, torch.cuda.current_stream(device).cuda_stream)
    buf = _status_ws.get(key)
    if buf is None:
        buf = torch.zeros(64, dtype=torch.int32, device=device)
        _status_ws[key] = buf
    return buf


def _check(cond: bool, msg: str) -> None:
    if not cond:
        raise RuntimeError(msg)


def _check_cuda(*ts) -> None:
    _check(all(t.is_cuda for t in ts), "superl8_b200: all inputs (incl. scales) must be CUDA tensors")
    _check(all(t.device == ts[0].device for t in ts), "superl8_b200: all inputs must be on the same device")


def device_status(device=None) -> int:
    """Synchronises and returns the device status word of the current stream's
    status buffer (0, or the DEVICE_TIMEOUT code when a bounded wait expired)."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    lib = _lib.load()
    rc = lib.sl8_read_device_status(_ptr(_status_buffer(device)), _stream(device))
    ws = _decode_ws.get((device.index, torch.cuda.current_stream(device).cuda_stream))
    if rc == 0 and ws is not None:
        rc = lib.sl8_read_device_status(_ptr(ws), _stream(device))
    bws = _bwd_ws.get((device.index, torch.cuda.current_stream(device).cuda_stream))
    if rc == 0 and bws is not None:
        rc = lib.sl8_read_device_status(_ptr(bws), _stream(device))
    if rc == 0 and _ext is not None:
        rc = int(_ext.device_status(torch.empty(0, device=device)))
    return rc


def quantize_i8_rowwise(x: torch.Tensor):
    """x [M, K] fp16/bf16/fp32 -> (q int8 [M, K], scale fp32 [M]).
    Reference binding: csrc/fni8_api.cpp:286-291; op csrc/kernel/quant_rowwise.cu:84-121."""
    if _compiled():
        r = _ext.quantize_i8_rowwise(x)
        _lib.launches += 1 if x.numel() else 0
        return r
    _check(x.is_cuda, "superl8_b200 quantize_i8_rowwise: x must be a CUDA tensor")
    _check(x.dim() == 2, "superl8_b200 quantize_i8_rowwise: expect [M, K]")
    _check(x.dtype in _DTYPE, "superl8_b200 quantize_i8_rowwise: x must be float16, bfloat16 or float32")
    x = x.contiguous()
    M, K = x.shape
    q = torch.empty((M, K), dtype=torch.int8, device=x.device)
    scale = torch.empty((M,), dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        rc = _lib.load().sl8_quantize_i8_rowwise(_ptr(x), _DTYPE[x.dtype], M, K, _ptr(q), _ptr(scale), _stream(x.device))
    _lib.check(rc, "quantize_i8_rowwise", 1)
    return q, scale


def _fwd_checks(q, q_scale, k, k_scale, v, what):
    _check_cuda(q, q_scale, k, k_scale, v)
    _check(q.dtype == torch.int8 and k.dtype == torch.int8, f"{what}: q/k must be int8")
    _check(q_scale.dtype == torch.float32 and k_scale.dtype == torch.float32, f"{what}: scales must be float32")
    _check(q.dim() == 4 and k.dim() == 4 and v.dim() == 4, f"{what}: expect [B,H,S,D]")
    _check(all(t.is_contiguous() for t in (q, q_scale, k, k_scale, v)), f"{what}: inputs must be contiguous")
    B, H, M, D = q.shape
    Hkv, N = k.shape[1], k.shape[2]
    _check(k.shape[0] == B and v.shape[0] == B and v.shape[1] == Hkv, f"{what}: batch/head mismatch")
    _check(Hkv > 0 and H % Hkv == 0, f"{what}: H_q must be divisible by H_kv (GQA)")
    _check(k.shape[3] == D and v.shape[3] == D and v.shape[2] == N, f"{what}: K/V shape mismatch")
    _check(q_scale.numel() == B * H * M and k_scale.numel() == B * Hkv * N, f"{what}: scale shape mismatch")
    return B, H, Hkv, M, N, D


def _gate_args(gate_flag, gate_want, device, what):
    if gate_flag is None:
        return dict(gate_flag=None, gate_want=0)
    _check(gate_flag.is_cuda and gate_flag.device == device and gate_flag.dtype == torch.int32 and gate_flag.numel() >= 1,
           f"{what}: gate_flag must be an int32 CUDA tensor on the inputs' device")
    return dict(gate_flag=gate_flag.data_ptr(), gate_want=int(bool(gate_want)))


def _run_fwd(q, q_scale, k, k_scale, v, causal, want_lse, window_left, seqlens_q=None, seqlens_k=None,
             backend=_lib.SL8_BACKEND_AUTO, out=None, gate_flag=None, gate_want=False):
    what = "superl8_b200"
    B, H, Hkv, M, N, D = _fwd_checks(q, q_scale, k, k_scale, v, what)
    _check(v.dtype in (torch.float16, torch.bfloat16), f"{what}: v must be float16 or bfloat16")
    _check(D in (32, 64, 72, 80, 128, 256), f"{what}: head dim must be 32/64/72/80/128/256, got {D}")
    if out is None:
        out = torch.empty((B, H, M, D), dtype=v.dtype, device=v.device)
    else:
        _check(out.shape == (B, H, M, D) and out.dtype == v.dtype and out.device == v.device and out.is_contiguous(),
               f"{what}: out must be a contiguous [B,H,M,D] tensor of v's dtype on v's device")
    lse = torch.empty((B, H, M) if want_lse else (0,), dtype=torch.float32, device=q.device)
    if M == 0 or B == 0 or H == 0:
        return out, lse
    for s in (seqlens_q, seqlens_k):
        if s is not None:
            _check(s.is_cuda and s.dtype == torch.int32 and s.numel() == B and s.is_contiguous(),
                   f"{what}: seqlens must be contiguous int32 [B] CUDA tensors")
    p = _lib.FwdParams(
        q=q.data_ptr(), q_scale=q_scale.data_ptr(), k=k.data_ptr(), k_scale=k_scale.data_ptr(), v=v.data_ptr(),
        out=out.data_ptr(), lse=lse.data_ptr() if want_lse else None,
        seqlens_q=None if seqlens_q is None else seqlens_q.data_ptr(),
        seqlens_k=None if seqlens_k is None else seqlens_k.data_ptr(),
        B=B, Hq=H, Hkv=Hkv, M=M, N=N, D=D, v_dtype=_DTYPE[v.dtype], causal=int(bool(causal)),
        window_left=int(window_left), backend=int(backend), **_gate_args(gate_flag, gate_want, q.device, what))
    with torch.cuda.device(q.device):
        ws = _status_buffer(q.device)
        rc = _lib.load().sl8_attn_int8_fwd(C.byref(p), _ptr(ws), ws.numel() * 4, _stream(q.device))
    _lib.check(rc, "attn_int8_fwd", 1)
    return out, lse


def attn_int8_fwd(q, q_scale, k, k_scale, v, causal=False, window_left=-1, *, seqlens_q=None, seqlens_k=None,
                  backend=_lib.SL8_BACKEND_AUTO, out=None, gate_flag=None, gate_want=False):
    """Reference binding csrc/fni8_api.cpp:225-229 (op csrc/kernel/attn_int8_fwd.cu:185-190).
    ``out`` (optional) receives the result; ``gate_flag`` (int32 CUDA tensor, optional) makes the
    launch conditional on the device: the kernel works only if (flag != 0) == gate_want."""
    if (_compiled() and seqlens_q is None and seqlens_k is None and backend == _lib.SL8_BACKEND_AUTO and out is None
            and gate_flag is None):
        r = _ext.attn_int8_fwd(q, q_scale, k, k_scale, v, bool(causal), int(window_left))
        _lib.launches += 1 if r.numel() else 0
        return r
    return _run_fwd(q, q_scale, k, k_scale, v, causal, False, window_left, seqlens_q, seqlens_k, backend,
                    out, gate_flag, gate_want)[0]


def attn_int8_fwd_train(q, q_scale, k, k_scale, v, causal=False, *, backend=_lib.SL8_BACKEND_AUTO):
    """Also returns the natural-log LSE.  Reference binding csrc/fni8_api.cpp:230-233."""
    if _compiled() and backend == _lib.SL8_BACKEND_AUTO:
        r = _ext.attn_int8_fwd_train(q, q_scale, k, k_scale, v, bool(causal))
        _lib.launches += 1 if r[0].numel() else 0
        return r
    return _run_fwd(q, q_scale, k, k_scale, v, causal, True, -1, None, None, backend)


def attn_int8_fwd_fused(q, k, v, causal=False, scale=None, window_left=-1, *, seqlens_q=None, seqlens_k=None,
                        gate=True, ratio_threshold=12.0):
    """attn_int8_fwd from 16-bit q, k, v [B, H, S, D] in ONE library call (sl8_attn_int8_fwd_fused):
    gate, Q / K prologue and both candidate kernels queued back to back, the gate decided on the
    device.  Returns (out, flag): flag is an int32 [1] device tensor, non-zero when the
    full-precision kernel produced ``out``.  D in {64, 128, 256}, one dtype, N > 0."""
    what = "superl8_b200 fused fwd"
    _check_cuda(q, k, v)
    _check(q.dtype in (torch.float16, torch.bfloat16), f"{what}: q must be float16 or bfloat16")
    _check(k.dtype == q.dtype and v.dtype == q.dtype, f"{what}: q, k, v must share one dtype")
    _check(q.dim() == 4 and k.dim() == 4 and v.dim() == 4, f"{what}: expect [B,H,S,D]")
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    B, H, M, D = q.shape
    Hkv, N = k.shape[1], k.shape[2]
    _check(k.shape[0] == B and v.shape[0] == B and v.shape[1] == Hkv, f"{what}: batch/head mismatch")
    _check(Hkv > 0 and H % Hkv == 0, f"{what}: H_q must be divisible by H_kv (GQA)")
    _check(k.shape[3] == D and v.shape[3] == D and v.shape[2] == N, f"{what}: K/V shape mismatch")
    _check(D in (64, 128, 256), f"{what}: head dim must be 64/128/256, got {D}")
    for s_ in (seqlens_q, seqlens_k):
        if s_ is not None:
            _check(s_.is_cuda and s_.dtype == torch.int32 and s_.numel() == B and s_.is_contiguous(),
                   f"{what}: seqlens must be contiguous int32 [B] CUDA tensors")
    out = torch.empty((B, H, M, D), dtype=v.dtype, device=v.device)
    sc = (1.0 / math.sqrt(D)) if scale is None else float(scale)
    status = _status_buffer(q.device)      # the stream's shared status word: device_status() reads it
    flag = torch.empty(1, dtype=torch.int32, device=q.device)   # zeroed by the call; outlives the workspace
    p = _lib.FusedFwdParams(
        q=q.data_ptr(), k=k.data_ptr(), v=v.data_ptr(), out=out.data_ptr(), device_status=status.data_ptr(),
        gate_flag=flag.data_ptr(),
        seqlens_q=None if seqlens_q is None else seqlens_q.data_ptr(),
        seqlens_k=None if seqlens_k is None else seqlens_k.data_ptr(),
        B=B, Hq=H, Hkv=Hkv, M=M, N=N, D=D, dtype=_DTYPE[q.dtype], causal=int(bool(causal)),
        window_left=int(window_left), ratio_threshold=float(ratio_threshold) if gate else 0.0, softmax_scale=sc)
    lib = _lib.load()
    with torch.cuda.device(q.device):
        nbytes = int(lib.sl8_attn_int8_fwd_fused_workspace(C.byref(p)))
        ws = torch.empty(nbytes, dtype=torch.uint8, device=q.device)
        rc = lib.sl8_attn_int8_fwd_fused(C.byref(p), _ptr(ws), nbytes, _stream(q.device))
    _lib.check(rc, "attn_int8_fwd_fused",
               (2 + _lib.k_prologue_launches(_DTYPE[k.dtype], B * Hkv, N, D) + (1 if gate else 0)) if out.numel() else 0)
    return out, flag


def qk_logits_i32(q_i8: torch.Tensor, k_i8: torch.Tensor) -> torch.Tensor:
    """int32 q[M,D] . k[N,D]^T on the tcgen05 kind::i8 tile path (no reference op; see the header)."""
    _check(q_i8.is_cuda and k_i8.is_cuda and q_i8.dtype == torch.int8 and k_i8.dtype == torch.int8,
           "superl8_b200 qk_logits_i32: q/k must be int8 CUDA tensors")
    _check(q_i8.dim() == 2 and k_i8.dim() == 2 and q_i8.shape[1] == k_i8.shape[1], "superl8_b200 qk_logits_i32: expect [M,D],[N,D]")
    q_i8, k_i8 = q_i8.contiguous(), k_i8.contiguous()
    M, D = q_i8.shape
    N = k_i8.shape[0]
    _check(D in (64, 128, 256), f"superl8_b200 qk_logits_i32: head dim must be 64/128/256, got {D}")
    s = torch.empty((M, N), dtype=torch.int32, device=q_i8.device)
    with torch.cuda.device(q_i8.device):
        ws = _status_buffer(q_i8.device)
        rc = _lib.load().sl8_qk_logits_i32(_ptr(q_i8), _ptr(k_i8), M, N, D, _ptr(s), _ptr(ws), ws.numel() * 4,
                                           _stream(q_i8.device))
    _lib.check(rc, "qk_logits_i32", 1)
    return s


def tensor_peak(kind_i8: bool, iters: int = 4096, device=None, n_cols: int = 256) -> float:
    """Measured tensor-pipe peak in T(FL)OP/s for kind::i8 (or kind::f16): times the probe launch
    with CUDA events after one warm-up launch.  ``n_cols`` (64, 128, 256) = N of the instruction."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    lib = _lib.load()
    ops = C.c_double(0.0)
    with torch.cuda.device(device):
        ws = _status_buffer(device)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for i in range(2):
            if i == 1:
                e0.record()
            rc = lib.sl8_tensor_peak_probe_n(int(bool(kind_i8)), int(n_cols), int(iters), C.byref(ops), _ptr(ws),
                                             ws.numel() * 4, _stream(device))
            _lib.check(rc, "tensor_peak_probe", 1)
        e1.record()
        torch.cuda.synchronize(device)
    return ops.value / (e0.elapsed_time(e1) * 1e-3) / 1e12


def attn_fp16_fwd(q, k, v, causal=False, scale=None, window_left=-1, mask=None, *, seqlens_q=None, seqlens_k=None,
                  backend=_lib.SL8_BACKEND_AUTO, want_lse=False, out=None, gate_flag=None, gate_want=False):
    """Full-precision forward.  Reference binding csrc/fni8_api.cpp:234-244.  ``want_lse``: also
    return the natural-log row sums [B, H, M] (what the backward consumes).  ``out`` / ``gate_flag`` /
    ``gate_want``: as in attn_int8_fwd (conditional launch decided on the device)."""
    what = "superl8_b200 fp16 fwd"
    if (_compiled() and seqlens_q is None and seqlens_k is None and backend == _lib.SL8_BACKEND_AUTO and out is None
            and gate_flag is None):
        sc_ = None if scale is None else float(scale)
        if want_lse and mask is None and window_left < 0:
            r = _ext.attn_fp16_fwd_train(q, k, v, bool(causal), sc_)
            _lib.launches += 1 if r[0].numel() else 0
            return r
        if not want_lse:
            r = _ext.attn_fp16_fwd(q, k, v, bool(causal), sc_, int(window_left), mask)
            _lib.launches += 1 if r.numel() else 0
            return r
    _check_cuda(q, k, v)
    _check(q.dtype in (torch.float16, torch.bfloat16), f"{what}: q must be float16 or bfloat16")
    _check(k.dtype == q.dtype and v.dtype == q.dtype, f"{what}: q, k, v must share one dtype")
    _check(q.dim() == 4 and k.dim() == 4 and v.dim() == 4, f"{what}: expect [B,H,S,D]")
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    B, H, M, D = q.shape
    Hkv, N = k.shape[1], k.shape[2]
    mk = dict(mask=None, mask_stride_b=0, mask_stride_h=0, mask_stride_m=0, mask_stride_n=0)
    if mask is not None:
        _check(mask.is_cuda and mask.device == q.device, f"{what}: mask must be a CUDA tensor on q's device")
        _check(mask.dtype == q.dtype, f"{what}: mask dtype must match q/k/v")
        _check(mask.dim() == 4, f"{what}: mask must be 4-D [B|1, H|1, M, N]")
        _check(mask.shape[2] == M and mask.shape[3] == N, f"{what}: mask trailing dims must be [M,N]")
        _check(mask.shape[0] in (B, 1) and mask.shape[1] in (H, 1), f"{what}: mask leading dims must broadcast to [B,H]")
        # indexed in place: a broadcast [B,1,M,N] view is never expanded (zero stride on size-1 axes)
        mk = dict(mask=mask.data_ptr(), mask_stride_b=0 if mask.shape[0] == 1 else mask.stride(0),
                  mask_stride_h=0 if mask.shape[1] == 1 else mask.stride(1),
                  mask_stride_m=mask.stride(2), mask_stride_n=mask.stride(3))
    _check(k.shape[0] == B and v.shape[0] == B and v.shape[1] == Hkv, f"{what}: batch/head mismatch")
    _check(Hkv > 0 and H % Hkv == 0, f"{what}: H_q must be divisible by H_kv (GQA)")
    _check(k.shape[3] == D and v.shape[3] == D and v.shape[2] == N, f"{what}: K/V shape mismatch")
    _check(D in (32, 64, 72, 80, 128, 256), f"{what}: head dim must be 32/64/72/80/128/256, got {D}")
    if out is None:
        out = torch.empty((B, H, M, D), dtype=v.dtype, device=v.device)
    else:
        _check(out.shape == (B, H, M, D) and out.dtype == v.dtype and out.device == v.device and out.is_contiguous(),
               f"{what}: out must be a contiguous [B,H,M,D] tensor of v's dtype on v's device")
    lse = torch.empty((B, H, M), dtype=torch.float32, device=v.device) if want_lse else None
    if out.numel() == 0:
        return (out, lse) if want_lse else out
    sc = (1.0 / math.sqrt(D)) if scale is None else float(scale)
    p = _lib.Fp16FwdParams(
        q=q.data_ptr(), k=k.data_ptr(), v=v.data_ptr(), out=out.data_ptr(), lse=None if lse is None else lse.data_ptr(),
        seqlens_q=None if seqlens_q is None else seqlens_q.data_ptr(),
        seqlens_k=None if seqlens_k is None else seqlens_k.data_ptr(),
        B=B, Hq=H, Hkv=Hkv, M=M, N=N, D=D, dtype=_DTYPE[q.dtype], causal=int(bool(causal)),
        window_left=int(window_left), softmax_scale=sc, backend=int(backend), **mk,
        **_gate_args(gate_flag, gate_want, q.device, what))
    with torch.cuda.device(q.device):
        ws = _status_buffer(q.device)
        rc = _lib.load().sl8_attn_fp16_fwd(C.byref(p), _ptr(ws), ws.numel() * 4, _stream(q.device))
    _lib.check(rc, "attn_fp16_fwd", 1)
    return (out, lse) if want_lse else out


def _decode_workspace(device, nbytes: int) -> torch.Tensor:
    key = (device.index, torch.cuda.current_stream(device).cuda_stream)
    buf = _decode_ws.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = torch.empty(nbytes, dtype=torch.uint8, device=device)
        buf[:256].zero_()
        _decode_ws[key] = buf
    return buf


def attn_int8_decode(q, q_scale, k, k_scale, v, num_splits=-1, *, context_lens=None):
    """Reference binding csrc/fni8_api.cpp:260-263 (op csrc/kernel/attn_decode.cu:163-240)."""
    what = "superl8_b200 decode"
    if _compiled() and context_lens is None:
        r = _ext.attn_int8_decode(q, q_scale, k, k_scale, v, int(num_splits))
        _lib.launches += 2 if (r.numel() and k.shape[2] > 0) else 0
        return r
    B, H, Hkv, M, N, D = _fwd_checks(q, q_scale, k, k_scale, v, what)
    _check(v.dtype == torch.float16, f"{what}: v must be float16")
    _check(M == 1, f"{what}: query length M must be 1 (decode)")
    _check(D in (32, 64, 128, 256), f"{what}: head dim must be 32/64/128/256, got {D}")
    num_splits = int(num_splits)
    _check(num_splits != 0, f"{what}: num_splits=0 is invalid; use -1 for auto or 1..256")
    if num_splits < 0:
        num_splits = -1
    _check(num_splits <= 256, f"{what}: num_splits must be 1..256, got {num_splits}")
    if context_lens is not None:
        _check(context_lens.is_cuda and context_lens.dtype == torch.int32 and context_lens.numel() == B
               and context_lens.is_contiguous(), f"{what}: context_lens must be a contiguous int32 [B] CUDA tensor")
    out = torch.empty((B, H, 1, D), dtype=v.dtype, device=v.device)
    if out.numel() == 0:
        return out
    p = _lib.DecodeParams(
        q=q.data_ptr(), q_scale=q_scale.data_ptr(), k=k.data_ptr(), k_scale=k_scale.data_ptr(), v=v.data_ptr(),
        out=out.data_ptr(), context_lens=None if context_lens is None else context_lens.data_ptr(),
        B=B, Hq=H, Hkv=Hkv, N=N, D=D, num_splits=num_splits)
    lib = _lib.load()
    with torch.cuda.device(q.device):
        ws = _decode_workspace(q.device, int(lib.sl8_attn_int8_decode_workspace(C.byref(p))))
        rc = lib.sl8_attn_int8_decode(C.byref(p), _ptr(ws), ws.numel(), _stream(q.device))
    _lib.check(rc, "attn_int8_decode", 2 if N > 0 else 0)
    return out


def attn_w8a8_fwd(q, q_scale, k, k_scale, v, v_scale, causal=False, causal_diag=0, per_warp_quant=True, *,
                  backend=None):
    """Full-W8A8 forward (int8 Q.K^T and int8 P.V).  Reference binding csrc/fni8_api.cpp:249-255
    (op csrc/kernel/attn_w8a8_fwd.cu:72-160): v int8 [B, Hkv, N, D], v_scale fp32 [B, Hkv, D];
    returns fp16 [B, Hq, M, D].  ``backend`` (an extension): None picks the tensor-memory kernel
    where it serves the call (D in 64/128/256, N > 0, causal diagonal at the sequence end) and the
    mma.sync kernel otherwise; SL8_BACKEND_TCGEN05 / SL8_BACKEND_MMA force one."""
    what = "superl8_b200 w8a8"
    _check(v.is_cuda and v.dtype == torch.int8, f"{what}: q/k/v must be int8")
    _check(v_scale.is_cuda and v_scale.dtype == torch.float32, f"{what}: scales must be float32")
    B, H, Hkv, M, N, D = _fwd_checks(q, q_scale, k, k_scale, v, what)
    _check(v_scale.is_contiguous() and v_scale.numel() == B * Hkv * D, f"{what}: scale shape mismatch")
    _check(D in (32, 64, 128, 256), f"{what}: head dim must be 32/64/128/256, got {D}")
    out = torch.empty((B, H, M, D), dtype=torch.float16, device=q.device)
    if out.numel() == 0:
        return out
    p = _lib.W8A8Params(q=q.data_ptr(), q_scale=q_scale.data_ptr(), k=k.data_ptr(), k_scale=k_scale.data_ptr(),
                        v=v.data_ptr(), v_scale=v_scale.data_ptr(), out=out.data_ptr(), B=B, Hq=H, Hkv=Hkv, M=M, N=N,
                        D=D, causal=int(bool(causal)), causal_diag=int(causal_diag), per_warp_quant=int(bool(per_warp_quant)))
    tc_ok = D in (64, 128, 256) and N > 0 and (not causal or int(causal_diag) == N - M)
    _check(backend in (None, _lib.SL8_BACKEND_TCGEN05, _lib.SL8_BACKEND_MMA), f"{what}: unknown backend {backend}")
    _check(tc_ok or backend != _lib.SL8_BACKEND_TCGEN05, f"{what}: the tensor-memory kernel does not serve this call")
    lib = _lib.load()
    with torch.cuda.device(q.device):
        if tc_ok and backend != _lib.SL8_BACKEND_MMA:
            ws = torch.empty(int(lib.sl8_attn_w8a8_fwd_tc_workspace(C.byref(p))), dtype=torch.uint8, device=q.device)
            rc = lib.sl8_attn_w8a8_fwd_tc(C.byref(p), _ptr(ws), ws.numel(), _stream(q.device))
        else:
            rc = lib.sl8_attn_w8a8_fwd(C.byref(p), _stream(q.device))
    _lib.check(rc, "attn_w8a8_fwd", 1)
    return out


def attn_int8_decode_kv8(q, q_scale, k, k_scale, v_i8, v_scale, num_splits=-1, *, context_lens=None):
    """Decode against an int8 K / int8 V cache.  Reference binding `attn_int8_decode_kv8`
    (kernel csrc/include/attn_decode.cuh:141-224): v_i8 int8 [B, Hkv, N, D], v_scale fp32
    [B, Hkv, D] (one scale per channel); everything else as attn_int8_decode."""
    what = "superl8_b200 decode kv8"
    _check(v_i8.is_cuda and v_i8.dtype == torch.int8, f"{what}: v must be an int8 CUDA tensor")
    _check(v_scale.is_cuda and v_scale.dtype == torch.float32, f"{what}: v_scale must be a float32 CUDA tensor")
    B, H, Hkv, M, N, D = _fwd_checks(q, q_scale, k, k_scale, v_i8, what)
    _check(M == 1, f"{what}: query length M must be 1 (decode)")
    _check(D in (32, 64, 128, 256), f"{what}: head dim must be 32/64/128/256, got {D}")
    _check(v_scale.numel() == B * Hkv * D, f"{what}: v_scale must be per-channel [B,H_kv,D]")
    num_splits = int(num_splits)
    _check(num_splits != 0, f"{what}: num_splits=0 is invalid; use -1 for auto or 1..256")
    if num_splits < 0:
        num_splits = -1
    _check(num_splits <= 256, f"{what}: num_splits must be 1..256, got {num_splits}")
    if context_lens is not None:
        _check(context_lens.is_cuda and context_lens.dtype == torch.int32 and context_lens.numel() == B
               and context_lens.is_contiguous(), f"{what}: context_lens must be a contiguous int32 [B] CUDA tensor")
    out = torch.empty((B, H, 1, D), dtype=torch.float16, device=q.device)
    if out.numel() == 0:
        return out
    v_i8, v_scale = v_i8.contiguous(), v_scale.contiguous()
    p = _lib.DecodeParams(
        q=q.data_ptr(), q_scale=q_scale.data_ptr(), k=k.data_ptr(), k_scale=k_scale.data_ptr(), v=v_i8.data_ptr(),
        out=out.data_ptr(), context_lens=None if context_lens is None else context_lens.data_ptr(),
        B=B, Hq=H, Hkv=Hkv, N=N, D=D, num_splits=num_splits)
    lib = _lib.load()
    with torch.cuda.device(q.device):
        ws = _decode_workspace(q.device, int(lib.sl8_attn_int8_decode_workspace(C.byref(p))))
        rc = lib.sl8_attn_int8_decode_kv8(C.byref(p), v_scale.data_ptr(), _ptr(ws), ws.numel(), _stream(q.device))
    _lib.check(rc, "attn_int8_decode_kv8", 2 if N > 0 else 0)
    return out


def attn_int8_varlen(q, q_scale, k, k_scale, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, causal=False, *,
                     backend=_lib.SL8_BACKEND_AUTO):
    """Packed variable-length prefill.  Reference binding `attn_int8_varlen`
    (csrc/kernel/attn_varlen_fwd.cu:45-110): q / k int8 [total, H, D], scales fp32 [total, H],
    v fp16 [total_k, Hkv, D], cu_seqlens int32 [B + 1]; returns [total_q, Hq, D] in v's dtype."""
    what = "superl8_b200 varlen"
    for t in (q, k, v, q_scale, k_scale, cu_seqlens_q, cu_seqlens_k):
        _check(t.is_cuda, f"{what}: all inputs must be CUDA tensors")
        _check(t.device == q.device, f"{what}: all inputs must be on the same device")
    _check(q.dtype == torch.int8 and k.dtype == torch.int8, f"{what}: q/k must be int8")
    _check(q_scale.dtype == torch.float32 and k_scale.dtype == torch.float32, f"{what}: scales must be float32")
    _check(v.dtype in (torch.float16, torch.bfloat16), f"{what}: v must be float16 or bfloat16")
    _check(cu_seqlens_q.dtype == torch.int32 and cu_seqlens_k.dtype == torch.int32, f"{what}: cu_seqlens must be int32")
    _check(q.dim() == 3 and k.dim() == 3 and v.dim() == 3, f"{what}: expect [total,H,D]")
    _check(all(t.is_contiguous() for t in (q, k, v, q_scale, k_scale, cu_seqlens_q, cu_seqlens_k)),
           f"{what}: inputs must be contiguous")
    total_q, H, D = q.shape
    total_k, Hkv = k.shape[0], k.shape[1]
    B = cu_seqlens_q.numel() - 1
    _check(B >= 1 and cu_seqlens_k.numel() == B + 1, f"{what}: cu_seqlens mismatch")
    _check(Hkv > 0 and H % Hkv == 0, f"{what}: H_q must be divisible by H_kv (GQA)")
    _check(k.shape[2] == D and v.shape[2] == D and v.shape[1] == Hkv and v.shape[0] == total_k, f"{what}: K/V shape")
    _check(q_scale.numel() == total_q * H and k_scale.numel() == total_k * Hkv, f"{what}: scale shape mismatch")
    _check(D in (32, 64, 128), f"{what}: head dim must be 32/64/128, got {D}")
    out = torch.empty((total_q, H, D), dtype=v.dtype, device=v.device)
    if out.numel() == 0:
        return out
    p = _lib.VarlenParams(q=q.data_ptr(), q_scale=q_scale.data_ptr(), k=k.data_ptr(), k_scale=k_scale.data_ptr(),
                          v=v.data_ptr(), out=out.data_ptr(), cu_seqlens_q=cu_seqlens_q.data_ptr(),
                          cu_seqlens_k=cu_seqlens_k.data_ptr(), B=B, Hq=H, Hkv=Hkv, D=D, total_q=total_q,
                          total_k=total_k, max_seqlen_q=int(max_seqlen_q), v_dtype=_DTYPE[v.dtype],
                          causal=int(bool(causal)), backend=int(backend))
    with torch.cuda.device(q.device):
        ws = _status_buffer(q.device)
        rc = _lib.load().sl8_attn_int8_varlen(C.byref(p), _ptr(ws), ws.numel() * 4, _stream(q.device))
    _lib.check(rc, "attn_int8_varlen", 1)
    return out


def attn_bwd(q, k, v, o, do_, lse, scale, causal=False, *, backend=_lib.SL8_BACKEND_AUTO):
    """Reference binding csrc/fni8_api.cpp:256-259 (op csrc/kernel/attn_bwd.cu:62-109):
    (dq, dk, dv) of the attention with logits scale * q.k, from the forward's output ``o``, its
    natural-log row sums ``lse`` [B, Hq, M] and the output gradient ``do_``.  q, o, do_
    [B, Hq, M, D]; k, v [B, Hkv, N, D]; dk / dv are summed over the query heads of a KV head."""
    what = "superl8_b200 bwd"
    if _compiled() and backend == _lib.SL8_BACKEND_AUTO:
        r = _ext.attn_bwd(q, k, v, o, do_, lse, float(scale), bool(causal))
        _lib.launches += 3 if (q.numel() and k.numel()) else 0
        return r
    for t in (q, k, v, o, do_, lse):
        _check(t.is_cuda, f"{what}: all inputs must be CUDA")
        _check(t.device == q.device, f"{what}: all inputs must be on the same device")
    _check(q.dtype in (torch.float16, torch.bfloat16) and all(t.dtype == q.dtype for t in (k, v, o, do_)),
           f"{what}: q/k/v/o/do must be float16 (or all bfloat16)")
    _check(lse.dtype == torch.float32, f"{what}: lse must be float32")
    _check(all(t.dim() == 4 for t in (q, k, v, o, do_)), f"{what}: expect [B,H,S,D]")
    q, k, v, o, do_, lse = (t.contiguous() for t in (q, k, v, o, do_, lse))
    B, H, M, D = q.shape
    Hkv, N = k.shape[1], k.shape[2]
    _check(Hkv > 0 and H % Hkv == 0, f"{what}: H_q must be divisible by H_kv (GQA)")
    _check(D in (32, 64, 128), f"{what}: head dim must be 32/64/128, got {D}")
    _check(k.shape == v.shape and k.shape[0] == B and k.shape[3] == D, f"{what}: K/V shape mismatch")
    _check(o.shape == q.shape and do_.shape == q.shape, f"{what}: o/do must have q's shape")
    _check(lse.numel() == B * H * M, f"{what}: lse must be [B,H,M]")
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    p = _lib.BwdParams(q=q.data_ptr(), k=k.data_ptr(), v=v.data_ptr(), o=o.data_ptr(), dout=do_.data_ptr(),
                       lse=lse.data_ptr(), dq=dq.data_ptr(), dk=dk.data_ptr(), dv=dv.data_ptr(),
                       B=B, Hq=H, Hkv=Hkv, M=M, N=N, D=D, dtype=_DTYPE[q.dtype], causal=int(bool(causal)),
                       softmax_scale=float(scale), backend=int(backend))
    lib = _lib.load()
    with torch.cuda.device(q.device):
        nbytes = lib.sl8_attn_bwd_workspace(C.byref(p))
        ws = torch.empty(nbytes, dtype=torch.uint8, device=q.device)   # status word; D_m = sum_d dO.O per query row
        ws[:256].zero_()
        rc = lib.sl8_attn_bwd(C.byref(p), _ptr(ws), nbytes, _stream(q.device))
        _bwd_ws[(q.device.index, torch.cuda.current_stream(q.device).cuda_stream)] = ws
    _lib.check(rc, "attn_bwd", 3 if (M and N and q.numel() and k.numel()) else 0)
    return dq, dk, dv
