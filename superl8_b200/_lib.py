"""ctypes binding of ``libsuperl8_b200.so`` (declarations: ``include/superl8_b200.h``).

The library is the product; there is no Python or CPU implementation behind
it.  If it is missing, every kernel call raises (``Sl8LibraryMissing``), the
same way the reference's ``_MissingC`` stand-in does (reference
superl8/ops.py:12-31).
"""

from __future__ import annotations

import ctypes as C
from pathlib import Path

import os

LIB_PATH = Path(os.environ.get("SUPERL8_B200_LIB") or (Path(__file__).resolve().parent / "libsuperl8_b200.so"))

SL8_OK = 0
SL8_F16, SL8_BF16, SL8_F32 = 0, 1, 2
SL8_BACKEND_AUTO, SL8_BACKEND_TCGEN05, SL8_BACKEND_MMA, SL8_BACKEND_TCGEN05_2Q = 0, 1, 2, 3

ERR_BAD_HEAD_DIM = -1
ERR_BAD_DTYPE = -2
ERR_MISALIGNED = -3
ERR_BAD_NUM_SPLITS = -4
ERR_WORKSPACE = -5
ERR_BAD_SHAPE = -6
ERR_NULL = -7
ERR_CUDA = -8
ERR_DEVICE_TIMEOUT = -9
ERR_UNSUPPORTED = -10
ERR_TOO_LARGE = -11


class Sl8LibraryMissing(RuntimeError):
    pass


class FwdParams(C.Structure):
    _fields_ = [
        ("q", C.c_void_p), ("q_scale", C.c_void_p), ("k", C.c_void_p), ("k_scale", C.c_void_p),
        ("v", C.c_void_p), ("out", C.c_void_p), ("lse", C.c_void_p),
        ("seqlens_q", C.c_void_p), ("seqlens_k", C.c_void_p),
        ("B", C.c_int32), ("Hq", C.c_int32), ("Hkv", C.c_int32), ("M", C.c_int32), ("N", C.c_int32),
        ("D", C.c_int32), ("v_dtype", C.c_int32), ("causal", C.c_int32), ("window_left", C.c_int32),
        ("backend", C.c_int32), ("gate_flag", C.c_void_p), ("gate_want", C.c_int32),
    ]


class Fp16FwdParams(C.Structure):
    _fields_ = [
        ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("out", C.c_void_p), ("lse", C.c_void_p),
        ("seqlens_q", C.c_void_p), ("seqlens_k", C.c_void_p),
        ("B", C.c_int32), ("Hq", C.c_int32), ("Hkv", C.c_int32), ("M", C.c_int32), ("N", C.c_int32),
        ("D", C.c_int32), ("dtype", C.c_int32), ("causal", C.c_int32), ("window_left", C.c_int32),
        ("softmax_scale", C.c_float), ("backend", C.c_int32),
        ("mask", C.c_void_p), ("mask_stride_b", C.c_int64), ("mask_stride_h", C.c_int64),
        ("mask_stride_m", C.c_int64), ("mask_stride_n", C.c_int64),
        ("gate_flag", C.c_void_p), ("gate_want", C.c_int32),
    ]


class FusedFwdParams(C.Structure):
    _fields_ = [
        ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("out", C.c_void_p),
        ("seqlens_q", C.c_void_p), ("seqlens_k", C.c_void_p), ("gate_flag", C.c_void_p),
        ("device_status", C.c_void_p),
        ("B", C.c_int32), ("Hq", C.c_int32), ("Hkv", C.c_int32), ("M", C.c_int32), ("N", C.c_int32), ("D", C.c_int32),
        ("dtype", C.c_int32), ("causal", C.c_int32), ("window_left", C.c_int32),
        ("ratio_threshold", C.c_float), ("softmax_scale", C.c_double),
    ]


class DecodeParams(C.Structure):
    _fields_ = [
        ("q", C.c_void_p), ("q_scale", C.c_void_p), ("k", C.c_void_p), ("k_scale", C.c_void_p),
        ("v", C.c_void_p), ("out", C.c_void_p), ("context_lens", C.c_void_p),
        ("B", C.c_int32), ("Hq", C.c_int32), ("Hkv", C.c_int32), ("N", C.c_int32), ("D", C.c_int32),
        ("num_splits", C.c_int32),
    ]


class W8A8Params(C.Structure):
    _fields_ = [
        ("q", C.c_void_p), ("q_scale", C.c_void_p), ("k", C.c_void_p), ("k_scale", C.c_void_p),
        ("v", C.c_void_p), ("v_scale", C.c_void_p), ("out", C.c_void_p),
        ("B", C.c_int32), ("Hq", C.c_int32), ("Hkv", C.c_int32), ("M", C.c_int32), ("N", C.c_int32), ("D", C.c_int32),
        ("causal", C.c_int32), ("causal_diag", C.c_int32), ("per_warp_quant", C.c_int32),
    ]


class VarlenParams(C.Structure):
    _fields_ = [
        ("q", C.c_void_p), ("q_scale", C.c_void_p), ("k", C.c_void_p), ("k_scale", C.c_void_p),
        ("v", C.c_void_p), ("out", C.c_void_p), ("cu_seqlens_q", C.c_void_p), ("cu_seqlens_k", C.c_void_p),
        ("B", C.c_int32), ("Hq", C.c_int32), ("Hkv", C.c_int32), ("D", C.c_int32),
        ("total_q", C.c_int64), ("total_k", C.c_int64), ("max_seqlen_q", C.c_int32),
        ("v_dtype", C.c_int32), ("causal", C.c_int32), ("backend", C.c_int32),
    ]


class HostFwdParams(C.Structure):
    _fields_ = [
        ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("out", C.c_void_p), ("gate_flags", C.c_void_p),
        ("B", C.c_int32), ("Hq", C.c_int32), ("Hkv", C.c_int32), ("M", C.c_int32), ("N", C.c_int32), ("D", C.c_int32),
        ("dtype", C.c_int32), ("causal", C.c_int32), ("window_left", C.c_int32), ("ratio_threshold", C.c_float),
        ("softmax_scale", C.c_double), ("kv_heads_per_chunk", C.c_int32), ("slots", C.c_int32),
    ]


class BwdParams(C.Structure):
    _fields_ = [
        ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("o", C.c_void_p), ("dout", C.c_void_p),
        ("lse", C.c_void_p), ("dq", C.c_void_p), ("dk", C.c_void_p), ("dv", C.c_void_p),
        ("B", C.c_int32), ("Hq", C.c_int32), ("Hkv", C.c_int32), ("M", C.c_int32), ("N", C.c_int32), ("D", C.c_int32),
        ("dtype", C.c_int32), ("causal", C.c_int32), ("softmax_scale", C.c_float), ("backend", C.c_int32),
    ]


# name -> (restype, argtypes); every symbol declared in include/superl8_b200.h
SIGNATURES = {
    "sl8_abi_version": (C.c_int, []),
    "sl8_status_string": (C.c_char_p, [C.c_int]),
    "sl8_quantize_i8_rowwise": (C.c_int, [C.c_void_p, C.c_int, C.c_int64, C.c_int64, C.c_void_p, C.c_void_p, C.c_void_p]),
    "sl8_quant_q_prologue": (C.c_int, [C.c_void_p, C.c_int, C.c_int64, C.c_int64, C.c_float, C.c_float,
                                       C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "sl8_q_outlier_gate": (C.c_int, [C.c_void_p, C.c_int, C.c_int64, C.c_int64, C.c_float, C.c_void_p, C.c_void_p]),
    "sl8_k_mean_workspace": (C.c_size_t, [C.c_int64, C.c_int64, C.c_int64]),
    "sl8_k_mean": (C.c_int, [C.c_void_p, C.c_int, C.c_int64, C.c_int64, C.c_int64, C.c_void_p, C.c_int32,
                             C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]),
    "sl8_smooth_quant_k": (C.c_int, [C.c_void_p, C.c_int, C.c_int64, C.c_int64, C.c_int64, C.c_void_p,
                                     C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "sl8_hadamard_quant_rows": (C.c_int, [C.c_void_p, C.c_int, C.c_int64, C.c_int64, C.c_void_p, C.c_int64, C.c_float,
                                          C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "sl8_k_prologue_fused_ok": (C.c_int, [C.c_int, C.c_int64, C.c_int64, C.c_int64]),
    "sl8_k_prologue": (C.c_int, [C.c_void_p, C.c_int, C.c_int64, C.c_int64, C.c_int64, C.c_void_p, C.c_int32,
                                 C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "sl8_attn_int8_fwd_workspace": (C.c_size_t, [C.POINTER(FwdParams)]),
    "sl8_attn_int8_fwd": (C.c_int, [C.POINTER(FwdParams), C.c_void_p, C.c_size_t, C.c_void_p]),
    "sl8_qk_logits_i32": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_void_p,
                                    C.c_void_p, C.c_size_t, C.c_void_p]),
    "sl8_attn_fp16_fwd_workspace": (C.c_size_t, [C.POINTER(Fp16FwdParams)]),
    "sl8_attn_fp16_fwd": (C.c_int, [C.POINTER(Fp16FwdParams), C.c_void_p, C.c_size_t, C.c_void_p]),
    "sl8_attn_int8_fwd_fused_workspace": (C.c_size_t, [C.POINTER(FusedFwdParams)]),
    "sl8_attn_int8_fwd_fused": (C.c_int, [C.POINTER(FusedFwdParams), C.c_void_p, C.c_size_t, C.c_void_p]),
    "sl8_attn_int8_fwd_host_workspace": (C.c_size_t, [C.POINTER(HostFwdParams)]),
    "sl8_attn_int8_fwd_host_chunks": (C.c_int, [C.POINTER(HostFwdParams)]),
    "sl8_attn_int8_fwd_host": (C.c_int, [C.POINTER(HostFwdParams), C.c_void_p, C.c_size_t, C.c_void_p]),
    "sl8_attn_w8a8_fwd": (C.c_int, [C.POINTER(W8A8Params), C.c_void_p]),
    "sl8_attn_w8a8_fwd_tc_workspace": (C.c_size_t, [C.POINTER(W8A8Params)]),
    "sl8_attn_w8a8_fwd_tc": (C.c_int, [C.POINTER(W8A8Params), C.c_void_p, C.c_size_t, C.c_void_p]),
    "sl8_attn_int8_varlen": (C.c_int, [C.POINTER(VarlenParams), C.c_void_p, C.c_size_t, C.c_void_p]),
    "sl8_k_mean_packed": (C.c_int, [C.c_void_p, C.c_int, C.c_int64, C.c_int32, C.c_int64, C.c_void_p, C.c_int32,
                                    C.c_void_p, C.c_void_p]),
    "sl8_smooth_quant_k_packed": (C.c_int, [C.c_void_p, C.c_int, C.c_int64, C.c_int32, C.c_int64, C.c_void_p,
                                            C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "sl8_attn_bwd_workspace": (C.c_size_t, [C.POINTER(BwdParams)]),
    "sl8_attn_bwd": (C.c_int, [C.POINTER(BwdParams), C.c_void_p, C.c_size_t, C.c_void_p]),
    "sl8_choose_n_splits": (C.c_int, [C.c_int64, C.c_int64]),
    "sl8_attn_int8_decode_workspace": (C.c_size_t, [C.POINTER(DecodeParams)]),
    "sl8_attn_int8_decode": (C.c_int, [C.POINTER(DecodeParams), C.c_void_p, C.c_size_t, C.c_void_p]),
    "sl8_attn_int8_decode_kv8": (C.c_int, [C.POINTER(DecodeParams), C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]),
    "sl8_quantize_v_perchannel": (C.c_int, [C.c_void_p, C.c_int, C.c_int64, C.c_int64, C.c_int64, C.c_void_p,
                                            C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]),
    "sl8_attn_int8_decode_static": (C.c_int, [C.POINTER(DecodeParams), C.c_void_p, C.c_void_p]),
    "sl8_tensor_peak_probe": (C.c_int, [C.c_int, C.c_int, C.POINTER(C.c_double), C.c_void_p, C.c_size_t, C.c_void_p]),
    "sl8_tensor_peak_probe_n": (C.c_int, [C.c_int, C.c_int, C.c_int, C.POINTER(C.c_double), C.c_void_p, C.c_size_t, C.c_void_p]),
    "sl8_decode_static_status": (C.c_int, [C.c_void_p]),
    "sl8_wait_timeout_selftest": (C.c_int, [C.c_void_p, C.c_size_t, C.c_uint64, C.c_void_p]),
    "sl8_read_device_status": (C.c_int, [C.c_void_p, C.c_void_p]),
}

DECODE_STATIC_SCRATCH_BYTES = 32 << 20

_lib = None

# number of kernels of this library launched so far (each wrapper adds its own launches)
launches = 0


def load():
    """Returns the loaded library (loads it on first use)."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise Sl8LibraryMissing(
            f"{LIB_PATH} is not built, so no superl8_b200 kernel can run. "
            "Build it with `python -m superl8_b200.build` (needs nvcc; cross-compiles for sm_100a). "
            "There is no CPU fallback."
        )
    lib = C.CDLL(str(LIB_PATH))
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def k_prologue_launches(dtype_code: int, BH: int, N: int, D: int) -> int:
    """Kernels the K prologue launches for this shape: 1 (cluster kernel) or 3 (mean partial, finish, quantise)."""
    return 1 if load().sl8_k_prologue_fused_ok(int(dtype_code), int(BH), int(N), int(D)) else 3


def status_string(code: int) -> str:
    return load().sl8_status_string(int(code)).decode()


def check(code: int, what: str, kernels: int = 0) -> None:
    """Turns a non-zero status into the RuntimeError the reference's TORCH_CHECKs raise;
    on success books ``kernels`` launches."""
    global launches
    if code != SL8_OK:
        raise RuntimeError(f"superl8_b200 {what}: {status_string(code)} (status {code})")
    launches += kernels
