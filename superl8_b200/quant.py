"""Quantisation prologue of the attention path, with the reference's function
names and return conventions (reference superl8/quant/core.py), running on the
sm_100a kernels of ``libsuperl8_b200.so``.

Arithmetic contract: the reference's CUDA semantics -- scale = amax * float32(1/127)
(csrc/include/quant_rowwise.cuh:33-38), codes = clamp(rint(x / scale), +-127),
K smoothing rounded to K's own dtype, folded Q scale = scale * float32(softmax_scale * log2 e).
"""

from __future__ import annotations

import ctypes as C
import math

import torch

from . import _C, _lib

LOG2E = math.log2(math.e)
Q_MAX = 127.0
OUTLIER_RATIO_THRESHOLD = 12.0


def _require_cuda(t: torch.Tensor, what: str) -> None:
    if not t.is_cuda:
        raise RuntimeError(f"superl8_b200 {what}: tensor must be on a CUDA device (there is no CPU path)")


def quantize_int8_rowwise(x: torch.Tensor):
    """Symmetric per-row int8.  Returns (q int8 [..., d], scale fp32 [..., 1]).
    Reference: superl8/quant/core.py:47-62."""
    _require_cuda(x, "quantize_int8_rowwise")
    shape = x.shape
    q, scale = _C.quantize_i8_rowwise(x.reshape(-1, shape[-1]))
    return q.reshape(shape), scale.reshape(*shape[:-1], 1)


def dequantize_int8_rowwise(q: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    return q.float() * scale


def k_mean(k: torch.Tensor, seqlens_k: torch.Tensor | None = None) -> torch.Tensor:
    """fp32 mean over the keys, [..., N, D] -> [..., 1, D] (reference
    superl8/quant/core.py:29-44).  With ``seqlens_k`` (int32 [B]) sequence b is
    averaged over its first seqlens_k[b] keys only."""
    _require_cuda(k, "k_mean")
    k = k.contiguous()
    N, D = k.shape[-2], k.shape[-1]
    BH = k.numel() // max(N * D, 1) if N * D else int(math.prod(k.shape[:-2]))
    mean = torch.empty((*k.shape[:-2], 1, D), dtype=torch.float32, device=k.device)
    if mean.numel() == 0:
        return mean
    lib = _lib.load()
    hpb = k.shape[1] if (seqlens_k is not None and k.dim() == 4) else 1
    with torch.cuda.device(k.device):
        ws_bytes = int(lib.sl8_k_mean_workspace(BH, N, D))
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device=k.device)
        rc = lib.sl8_k_mean(k.data_ptr(), _C._DTYPE[k.dtype], BH, N, D,
                            None if seqlens_k is None else seqlens_k.data_ptr(), hpb,
                            mean.data_ptr(), ws.data_ptr(), ws_bytes, _C._stream(k.device))
    _lib.check(rc, "k_mean", 2 if N > 0 else 0)
    return mean


def smooth_k(k: torch.Tensor, seqlens_k: torch.Tensor | None = None):
    """Subtract K's per-channel mean over the keys.  Returns (k_smoothed, k_mean).
    Reference: superl8/quant/core.py:70-95."""
    mean = k_mean(k, seqlens_k)
    _k_i8, _k_scale, k_s = smooth_quantize_k(k, mean, want_smoothed=True)
    return k_s, mean


def smooth_quantize_k(k: torch.Tensor, mean: torch.Tensor, want_smoothed: bool = False):
    """One pass: k_s = dtype(float(k) - mean), then the row quantiser.
    Returns (k_i8, k_scale [..., N, 1], k_s or None)."""
    _require_cuda(k, "smooth_quantize_k")
    if k.dtype not in (torch.float16, torch.bfloat16):
        raise RuntimeError("superl8_b200 smooth_quantize_k: k must be float16 or bfloat16")
    k = k.contiguous()
    mean = mean.contiguous().float()
    N, D = k.shape[-2], k.shape[-1]
    BH = int(math.prod(k.shape[:-2]))
    k_i8 = torch.empty(k.shape, dtype=torch.int8, device=k.device)
    k_scale = torch.empty((*k.shape[:-1], 1), dtype=torch.float32, device=k.device)
    k_s = torch.empty_like(k) if want_smoothed else None
    if k.numel():
        with torch.cuda.device(k.device):
            rc = _lib.load().sl8_smooth_quant_k(k.data_ptr(), _C._DTYPE[k.dtype], BH, N, D, mean.data_ptr(),
                                                k_i8.data_ptr(), k_scale.data_ptr(),
                                                None if k_s is None else k_s.data_ptr(), _C._stream(k.device))
        _lib.check(rc, "smooth_quant_k", 1)
    return k_i8, k_scale, k_s


def k_prologue(k: torch.Tensor, seqlens_k: torch.Tensor | None = None, want_smoothed: bool = False):
    """K prologue: fp32 mean over the keys, k_s = dtype(float(k) - mean), row quantiser.  Returns
    (k_i8, k_scale [..., N, 1], k_mean [..., 1, D], k_s or None).  One launch (a thread-block cluster
    per (batch, kv-head) slab, K read from HBM once) where the library serves the shape, otherwise
    k_mean + smooth_quantize_k; both give the same bits."""
    _require_cuda(k, "k_prologue")
    if k.dtype not in (torch.float16, torch.bfloat16):
        raise RuntimeError("superl8_b200 k_prologue: k must be float16 or bfloat16")
    k = k.contiguous()
    N, D = k.shape[-2], k.shape[-1]
    BH = int(math.prod(k.shape[:-2]))
    lib = _lib.load()
    if k.numel() == 0 or not lib.sl8_k_prologue_fused_ok(_C._DTYPE[k.dtype], BH, N, D):
        mean = k_mean(k, seqlens_k)
        k_i8, k_scale, k_s = smooth_quantize_k(k, mean, want_smoothed)
        return k_i8, k_scale, mean, k_s
    mean = torch.empty((*k.shape[:-2], 1, D), dtype=torch.float32, device=k.device)
    k_i8 = torch.empty(k.shape, dtype=torch.int8, device=k.device)
    k_scale = torch.empty((*k.shape[:-1], 1), dtype=torch.float32, device=k.device)
    k_s = torch.empty_like(k) if want_smoothed else None
    hpb = k.shape[1] if (seqlens_k is not None and k.dim() == 4) else 1
    with torch.cuda.device(k.device):
        rc = lib.sl8_k_prologue(k.data_ptr(), _C._DTYPE[k.dtype], BH, N, D,
                                None if seqlens_k is None else seqlens_k.data_ptr(), hpb, mean.data_ptr(),
                                k_i8.data_ptr(), k_scale.data_ptr(), None if k_s is None else k_s.data_ptr(),
                                _C._stream(k.device))
    _lib.check(rc, "k_prologue", 1)
    return k_i8, k_scale, mean, k_s


def quantize_v_perchannel(v: torch.Tensor):
    """Symmetric int8 per CHANNEL of V, scale over the key axis (reference
    superl8/quant/core.py:98-110): returns (v_i8 [..., N, D], v_scale fp32 [..., 1, D])."""
    _require_cuda(v, "quantize_v_perchannel")
    if v.dtype not in (torch.float16, torch.bfloat16):
        raise RuntimeError("superl8_b200 quantize_v_perchannel: v must be float16 or bfloat16")
    v = v.contiguous()
    N, D = v.shape[-2], v.shape[-1]
    BH = int(math.prod(v.shape[:-2]))
    v_i8 = torch.empty(v.shape, dtype=torch.int8, device=v.device)
    v_scale = torch.empty((*v.shape[:-2], 1, D), dtype=torch.float32, device=v.device)
    if BH * D:
        lib = _lib.load()
        with torch.cuda.device(v.device):
            ws_bytes = int(lib.sl8_k_mean_workspace(BH, N, D))
            ws = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device=v.device)
            rc = lib.sl8_quantize_v_perchannel(v.data_ptr(), _C._DTYPE[v.dtype], BH, N, D, v_i8.data_ptr(),
                                               v_scale.data_ptr(), ws.data_ptr(), ws_bytes, _C._stream(v.device))
        _lib.check(rc, "quantize_v_perchannel", 3 if N > 0 else 1)
    return v_i8, v_scale


def varlen_smooth_quantize_k(k: torch.Tensor, cu_seqlens_k: torch.Tensor, want_smoothed: bool = False,
                             k_mean_override: torch.Tensor | None = None):
    """Packed keys [total, H, D]: per-sequence K mean (reference superl8/ops.py:268-315
    `_varlen_smooth_k`), then k_s = dtype(float(k) - mean of the token's own sequence) and the row
    quantiser, all on the device with no read of cu_seqlens on the host.  ``k_mean_override``
    (fp32 [B, H, D]) replaces the computed means (exact reproduction of another implementation's).
    Returns (k_i8 [total, H, D], k_scale [total, H, 1], k_mean fp32 [B, H, D], k_s or None)."""
    _require_cuda(k, "varlen_smooth_quantize_k")
    if k.dtype not in (torch.float16, torch.bfloat16):
        raise RuntimeError("superl8_b200 varlen_smooth_quantize_k: k must be float16 or bfloat16")
    if k.dim() != 3:
        raise RuntimeError("superl8_b200 varlen_smooth_quantize_k: expect [total,H,D]")
    k = k.contiguous()
    cu = cu_seqlens_k.contiguous()
    total, H, D = k.shape
    B = cu.numel() - 1
    if k_mean_override is not None:
        mean = k_mean_override.to(device=k.device, dtype=torch.float32).reshape(B, H, D).contiguous()
    else:
        mean = torch.zeros((B, H, D), dtype=torch.float32, device=k.device)
    k_i8 = torch.empty(k.shape, dtype=torch.int8, device=k.device)
    k_scale = torch.empty((total, H, 1), dtype=torch.float32, device=k.device)
    k_s = torch.empty_like(k) if want_smoothed else None
    if k.numel() and B > 0:
        lib = _lib.load()
        with torch.cuda.device(k.device):
            st = _C._stream(k.device)
            if k_mean_override is None:
                rc = lib.sl8_k_mean_packed(k.data_ptr(), _C._DTYPE[k.dtype], total, H, D, cu.data_ptr(), B,
                                           mean.data_ptr(), st)
                _lib.check(rc, "k_mean_packed", 1)
            rc = lib.sl8_smooth_quant_k_packed(k.data_ptr(), _C._DTYPE[k.dtype], total, H, D, cu.data_ptr(), B,
                                               mean.data_ptr(), k_i8.data_ptr(), k_scale.data_ptr(),
                                               None if k_s is None else k_s.data_ptr(), st)
            _lib.check(rc, "smooth_quant_k_packed", 1)
    return k_i8, k_scale, mean, k_s


def quantize_q(q: torch.Tensor, softmax_scale: float, want_gate: bool = False,
               ratio_threshold: float = OUTLIER_RATIO_THRESHOLD):
    """Q prologue in one pass: codes, folded scale [..., M, 1] and (optionally) the
    device flag of the outlier gate (int32 [1], non-zero = some row is dominated)."""
    _require_cuda(q, "quantize_q")
    q = q.contiguous()
    D = q.shape[-1]
    rows = q.numel() // D if D else 0
    q_i8 = torch.empty(q.shape, dtype=torch.int8, device=q.device)
    q_scale = torch.empty((*q.shape[:-1], 1), dtype=torch.float32, device=q.device)
    flag = torch.zeros(1, dtype=torch.int32, device=q.device) if want_gate else None
    if q.numel():
        fold = softmax_scale * LOG2E
        with torch.cuda.device(q.device):
            rc = _lib.load().sl8_quant_q_prologue(q.data_ptr(), _C._DTYPE[q.dtype], rows, D, C.c_float(fold),
                                                  C.c_float(ratio_threshold), q_i8.data_ptr(), q_scale.data_ptr(),
                                                  None, None if flag is None else flag.data_ptr(),
                                                  _C._stream(q.device))
        _lib.check(rc, "quant_q_prologue", 1)
    return q_i8, q_scale, flag


def q_outlier_flag(q: torch.Tensor, ratio_threshold: float = OUTLIER_RATIO_THRESHOLD) -> torch.Tensor:
    """Device flag (int32 [1], non-zero = some row of q is outlier dominated) from one read of q,
    nothing quantised: the gate the reference evaluates before it quantises."""
    _require_cuda(q, "q_outlier_flag")
    q = q.contiguous()
    D = q.shape[-1]
    rows = q.numel() // D if D else 0
    flag = torch.zeros(1, dtype=torch.int32, device=q.device)
    if q.numel():
        with torch.cuda.device(q.device):
            rc = _lib.load().sl8_q_outlier_gate(q.data_ptr(), _C._DTYPE[q.dtype], rows, D, C.c_float(ratio_threshold),
                                                flag.data_ptr(), _C._stream(q.device))
        _lib.check(rc, "q_outlier_gate", 1)
    return flag


def _capturing() -> bool:
    try:
        return bool(torch.cuda.is_current_stream_capturing())
    except Exception:
        return False


def detect_q_outlier_domination(q: torch.Tensor, *, ratio_threshold: float = OUTLIER_RATIO_THRESHOLD) -> bool:
    """True when any row of q has max|q| / (median|q| + 1e-10) > ratio_threshold.
    Skipped (False) while the stream is being captured into a CUDA graph, like the
    reference (superl8/quant/core.py:113-145): the answer needs a device->host read."""
    if _capturing():
        return False
    return bool(q_outlier_flag(q, ratio_threshold).item())


def _rotation_kernel_ok(x: torch.Tensor) -> bool:
    d = x.shape[-1]
    return x.is_cuda and x.dtype in (torch.float16, torch.bfloat16) and 32 <= d <= 1024 and d & (d - 1) == 0


def hadamard_quantize_rows(x: torch.Tensor, *, mean: torch.Tensor | None = None, fold: float = 1.0,
                           want_codes: bool = True, want_rotated: bool = False):
    """[smooth] -> Hadamard rotation -> [quantise] of the rows of x [..., N, D] in one kernel pass
    (sl8_hadamard_quant_rows): the rotate=True prologue of the reference (superl8/quant/core.py:186-194).
    ``mean`` fp32 [..., D] per slab of N rows (K), None for Q.  Returns (codes or None,
    scale [..., N, 1] * fold or None, rotated rows in x's dtype or None)."""
    _require_cuda(x, "hadamard_quantize_rows")
    if not _rotation_kernel_ok(x):
        raise RuntimeError("superl8_b200 hadamard_quantize_rows: float16 or bfloat16, power-of-two last dim in [32, 1024]")
    x = x.contiguous()
    D = x.shape[-1]
    rows = x.numel() // D
    q = torch.empty(x.shape, dtype=torch.int8, device=x.device) if want_codes else None
    scale = torch.empty((*x.shape[:-1], 1), dtype=torch.float32, device=x.device) if want_codes else None
    rot = torch.empty_like(x) if want_rotated else None
    if mean is not None:
        mean = mean.to(device=x.device, dtype=torch.float32).contiguous()
    if rows:
        with torch.cuda.device(x.device):
            rc = _lib.load().sl8_hadamard_quant_rows(
                x.data_ptr(), _C._DTYPE[x.dtype], rows, D, None if mean is None else mean.data_ptr(),
                x.shape[-2] if x.dim() >= 2 else 1, C.c_float(fold), None if q is None else q.data_ptr(),
                None if scale is None else scale.data_ptr(), None if rot is None else rot.data_ptr(), _C._stream(x.device))
        _lib.check(rc, "hadamard_quant_rows", 1)
    return q, scale, rot


def rotate_last(x: torch.Tensor) -> torch.Tensor:
    """Normalised Sylvester-Hadamard rotation of the last dim in fp32, cast back
    (reference superl8/quant/rotation.py:28-51): a Walsh-Hadamard butterfly in the row quantiser's
    registers for 16-bit CUDA tensors with a power-of-two last dim in [32, 1024], the reference's
    own matmul formula in torch otherwise (fp32 input, other sizes)."""
    d = x.shape[-1]
    if d & (d - 1):
        raise ValueError(f"Hadamard rotation needs a power-of-two last dim, got {d}")
    if _rotation_kernel_ok(x):
        return hadamard_quantize_rows(x, want_codes=False, want_rotated=True)[2]
    h = torch.ones(1, 1, device=x.device, dtype=torch.float32)
    while h.shape[0] < d:
        h = torch.cat([torch.cat([h, h], 1), torch.cat([h, -h], 1)], 0)
    return (x.float() @ (h / math.sqrt(d))).to(x.dtype)


def quantize_qk(q, k, *, softmax_scale: float | None = None, rotate: bool = False, k_mean_override=None,
                seqlens_k=None):
    """Returns (q_int8, q_scale[..., m, 1] folded, k_int8, k_scale[..., n, 1], k_mean[..., 1, d]).
    Reference: superl8/quant/core.py:164-196.  ``k_mean_override`` supplies the mean
    instead of computing it (the summation order of a mean is not portable bit for bit)."""
    if softmax_scale is None:
        softmax_scale = 1.0 / math.sqrt(q.shape[-1])
    if rotate and _rotation_kernel_ok(q) and _rotation_kernel_ok(k):
        # smoothing, rotation and quantisation of a row in one pass each for Q and K
        mean = k_mean(k, seqlens_k) if k_mean_override is None else k_mean_override
        k_i8, k_scale, _ = hadamard_quantize_rows(k, mean=mean.reshape(*k.shape[:-2], k.shape[-1]))
        q_i8, q_scale, _ = hadamard_quantize_rows(q, fold=softmax_scale * LOG2E)
        return q_i8, q_scale, k_i8, k_scale, mean
    if rotate:
        mean = k_mean(k, seqlens_k) if k_mean_override is None else k_mean_override
        _ki8, _ks, k_s = smooth_quantize_k(k, mean, want_smoothed=True)
        q = rotate_last(q)
        k_i8, k_scale = quantize_int8_rowwise(rotate_last(k_s))
    elif k_mean_override is not None:
        mean = k_mean_override
        k_i8, k_scale, _ = smooth_quantize_k(k, mean)
    else:
        k_i8, k_scale, mean, _ = k_prologue(k, seqlens_k)
    q_i8, q_scale, _ = quantize_q(q, softmax_scale)
    return q_i8, q_scale, k_i8, k_scale, mean
