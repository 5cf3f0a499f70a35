"""Helpers shared by the GPU tests: the reference-kernel checker library and input makers."""

import ctypes as C
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent.parent
REF_LIB_PATH = ROOT / "oracle" / "_ref" / "libref_kernels.so"
_ref = None


def ref_lib():
    """The reference's own CUDA kernels (oracle/_ref, built by oracle/build_ref.py), or None."""
    global _ref
    if _ref is None and REF_LIB_PATH.exists():
        _ref = C.CDLL(str(REF_LIB_PATH))
    return _ref


def _p(t):
    return C.c_void_p(t.data_ptr()) if t is not None else None


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


_DT = {torch.float16: 0, torch.bfloat16: 1, torch.float32: 2}


def ref_quantize(x):
    M, K = x.shape
    q = torch.empty((M, K), dtype=torch.int8, device=x.device)
    s = torch.empty((M,), dtype=torch.float32, device=x.device)
    rc = ref_lib().ref_quantize_i8_rowwise(_p(x), _DT[x.dtype], M, K, _p(q), _p(s), _stream())
    assert rc == 0
    return q, s


def ref_fwd(q_i8, q_scale, k_i8, k_scale, v, causal=False, window_left=-1, want_lse=False):
    B, Hq, M, D = q_i8.shape
    Hkv, N = k_i8.shape[1], k_i8.shape[2]
    out = torch.empty((B, Hq, M, D), dtype=v.dtype, device=v.device)
    lse = torch.empty((B, Hq, M), dtype=torch.float32, device=v.device) if want_lse else None
    rc = ref_lib().ref_attn_int8_fwd(_p(q_i8), _p(q_scale), _p(k_i8), _p(k_scale), _p(v), _DT[v.dtype], _p(out),
                                     _p(lse), int(causal), int(window_left), B, Hq, Hkv, M, N, D, _stream())
    assert rc == 0
    return (out, lse) if want_lse else out


def ref_decode(q_i8, q_scale, k_i8, k_scale, v, n_splits):
    B, Hq, _, D = q_i8.shape
    Hkv, N = k_i8.shape[1], k_i8.shape[2]
    out = torch.empty((B, Hq, 1, D), dtype=torch.float16, device=v.device)
    o_part = torch.empty((n_splits, B * Hq, D), dtype=torch.float32, device=v.device)
    m_part = torch.empty((n_splits, B * Hq), dtype=torch.float32, device=v.device)
    l_part = torch.empty((n_splits, B * Hq), dtype=torch.float32, device=v.device)
    rc = ref_lib().ref_attn_int8_decode(_p(q_i8), _p(q_scale), _p(k_i8), _p(k_scale), _p(v), _p(out), _p(o_part),
                                        _p(m_part), _p(l_part), B, Hq, Hkv, N, D, n_splits, _stream())
    assert rc == 0
    return out


def quantized_inputs(cfg, B, Hq, Hkv, M, D, N=None, dtype=torch.float16, device="cuda"):
    """Seeded fp inputs plus their oracle quantisation (CUDA scale rule), moved to the device.
    Returns dict with q,k,v (fp), q_i8,q_scale[B,Hq,M],k_i8,k_scale[B,Hkv,N] on device and CPU copies."""
    from oracle import oracle
    q, k, v = oracle.make_batch(cfg, B, Hq, Hkv, M, D, Sk=N, dtype=dtype)
    q_i8, q_scale, k_i8, k_scale, k_mean = oracle.quantize_qk(q, k)
    d = dict(q=q, k=k, v=v, q_i8=q_i8, q_scale=q_scale.squeeze(-1).contiguous(), k_i8=k_i8,
             k_scale=k_scale.squeeze(-1).contiguous(), k_mean=k_mean)
    d["dev"] = {n: t.to(device) for n, t in d.items()}
    return d


def ref_attn_int8_varlen(q_i8, q_scale, k_i8, k_scale, v, cu_q, cu_k, max_seqlen_q, causal):
    """The reference's packed variable-length kernel on the same int8 inputs."""
    total_q, Hq, D = q_i8.shape
    out = torch.empty((total_q, Hq, D), dtype=torch.float16, device=v.device)
    rc = ref_lib().ref_attn_int8_varlen(_p(q_i8), _p(q_scale), _p(k_i8), _p(k_scale), _p(v), _p(out), _p(cu_q), _p(cu_k),
                                        cu_q.numel() - 1, int(max_seqlen_q), Hq, k_i8.shape[1], D, int(causal), _stream())
    assert rc == 0
    return out


def ref_attn_int8_decode_kv8(q_i8, q_scale, k_i8, k_scale, v_i8, v_scale, n_splits):
    """The reference's int8-V split + combine kernels on the same inputs."""
    B, Hq, _, D = q_i8.shape
    Hkv, N = k_i8.shape[1], k_i8.shape[2]
    dev = q_i8.device
    out = torch.empty((B, Hq, 1, D), dtype=torch.float16, device=dev)
    o_part = torch.empty((n_splits, B * Hq, D), dtype=torch.float32, device=dev)
    m_part = torch.empty((n_splits, B * Hq), dtype=torch.float32, device=dev)
    l_part = torch.empty((n_splits, B * Hq), dtype=torch.float32, device=dev)
    rc = ref_lib().ref_attn_int8_decode_kv8(_p(q_i8), _p(q_scale), _p(k_i8), _p(k_scale), _p(v_i8), _p(v_scale), _p(out),
                                            _p(o_part), _p(m_part), _p(l_part), B, Hq, Hkv, N, D, n_splits, _stream())
    assert rc == 0
    return out


def ref_attn_w8a8_fwd(q_i8, q_scale, k_i8, k_scale, v_i8, v_scale, causal, causal_diag, per_warp):
    """The reference's full-W8A8 kernel on the same int8 inputs (D = 32, 64, 128)."""
    B, Hq, M, D = q_i8.shape
    Hkv, N = k_i8.shape[1], k_i8.shape[2]
    out = torch.empty((B, Hq, M, D), dtype=torch.float16, device=q_i8.device)
    rc = ref_lib().ref_attn_w8a8_fwd(_p(q_i8), _p(q_scale), _p(k_i8), _p(k_scale), _p(v_i8), _p(v_scale), _p(out),
                                     int(causal), int(causal_diag), int(per_warp), B, Hq, Hkv, M, N, D, _stream())
    assert rc == 0
    return out
