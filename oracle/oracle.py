"""CPU restatement of the reference's int8 attention path.  TEST INFRASTRUCTURE ONLY.

Only ``tests/``, ``__graft_entry__.smoke()`` and ``bench.py``'s CPU-baseline legs may
import this module; the product (``superl8_b200``) never does and has no CPU path.

Parity status: PINNED.  ``tests/test_oracle_golden.py`` checks every function here
against vectors produced by importing the reference's own Python code
(``tests/golden/make_golden.py`` -> ``tests/golden/*.npz``), and on a GPU box the
``-m gpu`` tests compare this repository's kernels with the reference's own CUDA kernels
compiled from its sources (``oracle/_ref``, helpers in ``tests/gpu_helpers.py``).

Two scale rules exist in the reference and both are restated:
  rule="cpu"   scale = amax / 127        (reference CPU branch, superl8/quant/core.py:58)
  rule="cuda"  scale = amax * f32(1/127) (reference CUDA kernel,
               csrc/include/quant_rowwise.cuh:33-38, 72) -- the parity target.
Everything is torch-on-CPU / numpy in fp32 with the reference's operation order.
"""

from __future__ import annotations

import math

import numpy as np
import torch

LOG2E = math.log2(math.e)  # reference superl8/quant/core.py:24
Q_MAX = 127.0              # reference superl8/quant/core.py:25
K_MEAN_CHUNK = 1024        # reference superl8/quant/core.py:26
DEC_NEG_INF = -1e30        # reference csrc/include/attn_decode.cuh:34


# --------------------------------------------------------------------------- quantiser

def quantize_rowwise(x: torch.Tensor, rule: str = "cuda"):
    """Reference superl8/quant/core.py:47-62 and csrc/include/quant_rowwise.cuh:42-92.
    Returns (q int8 [..., d], scale fp32 [..., 1])."""
    xf = x.detach().cpu().float()
    amax = xf.abs().amax(dim=-1, keepdim=True)
    if rule == "cuda":
        scale = amax * torch.tensor(np.float32(1.0) / np.float32(127.0))
    elif rule == "cpu":
        scale = amax / Q_MAX
    else:
        raise ValueError(rule)
    safe = torch.where(scale == 0, torch.ones_like(scale), scale)
    q = torch.round(xf / safe).clamp_(-Q_MAX, Q_MAX).to(torch.int8)
    return q, safe


def k_mean_fp32(k: torch.Tensor) -> torch.Tensor:
    """Reference superl8/quant/core.py:29-44: fp32 mean over keys, 1024-row partial sums
    when N > 1024.  (Summation order inside each partial is torch's own.)"""
    k = k.detach().cpu()
    n = k.shape[-2]
    if n <= K_MEAN_CHUNK:
        return torch.mean(k, dim=-2, keepdim=True, dtype=torch.float32)
    mean = torch.zeros((*k.shape[:-2], 1, k.shape[-1]), dtype=torch.float32)
    for start in range(0, n, K_MEAN_CHUNK):
        mean.add_(torch.sum(k[..., start:start + K_MEAN_CHUNK, :], dim=-2, keepdim=True, dtype=torch.float32))
    return mean.div_(n)


def smooth_k(k: torch.Tensor, mean: torch.Tensor | None = None):
    """Reference superl8/quant/core.py:70-95: k_s = dtype(fp32(k) - mean)."""
    k = k.detach().cpu()
    mean = k_mean_fp32(k) if mean is None else mean.detach().cpu().float()
    k_s = (k.float() - mean).to(k.dtype)
    return k_s, mean


def detect_q_outlier_domination(q: torch.Tensor, ratio_threshold: float = 12.0) -> bool:
    """Reference superl8/quant/core.py:113-145 (median = lower middle element)."""
    q_abs = q.detach().cpu().float().abs()
    row_max = q_abs.amax(dim=-1)
    row_med = q_abs.median(dim=-1).values
    return bool(((row_max / (row_med + 1e-10)) > ratio_threshold).any())


def outlier_rows(q: torch.Tensor, ratio_threshold: float = 12.0) -> torch.Tensor:
    q_abs = q.detach().cpu().float().abs()
    return (q_abs.amax(dim=-1) / (q_abs.median(dim=-1).values + 1e-10)) > ratio_threshold


def fold_scale(scale: torch.Tensor, softmax_scale: float) -> torch.Tensor:
    """Reference superl8/quant/core.py:195: fp32 tensor times a Python scalar."""
    return scale * (softmax_scale * LOG2E)


def hadamard_matrix(d: int) -> torch.Tensor:
    """Reference superl8/quant/rotation.py:28-38: the Sylvester-Hadamard matrix over sqrt(d), fp32."""
    assert d > 0 and d & (d - 1) == 0
    h = torch.ones(1, 1, dtype=torch.float32)
    while h.shape[0] < d:
        h = torch.cat([torch.cat([h, h], dim=1), torch.cat([h, -h], dim=1)], dim=0)
    return h / (d ** 0.5)


def rotate_last(x: torch.Tensor) -> torch.Tensor:
    """Reference superl8/quant/rotation.py:41-51: (x.float() @ M) cast back to x's dtype."""
    x = x.detach().cpu()
    return (x.float() @ hadamard_matrix(x.shape[-1])).to(x.dtype)


def quantize_qk(q, k, softmax_scale=None, rule: str = "cuda", k_mean=None, rotate: bool = False):
    """Reference superl8/quant/core.py:164-196; rotate: lines 186-190 (Q and the smoothed K rotated
    by the same Hadamard matrix before the row quantiser)."""
    if softmax_scale is None:
        softmax_scale = 1.0 / math.sqrt(q.shape[-1])
    k_s, mean = smooth_k(k, k_mean)
    if rotate:
        q, k_s = rotate_last(q), rotate_last(k_s)
    q_i8, q_scale = quantize_rowwise(q, rule)
    k_i8, k_scale = quantize_rowwise(k_s, rule)
    return q_i8, fold_scale(q_scale, softmax_scale), k_i8, k_scale, mean


# --------------------------------------------------------------------------- fp32 oracles

def _expand_kv(kf, vf, h_q):
    h_kv = kf.shape[1]
    if h_q != h_kv:
        assert h_q % h_kv == 0
        rep = h_q // h_kv
        kf = kf.repeat_interleave(rep, dim=1)
        vf = vf.repeat_interleave(rep, dim=1)
    return kf, vf


def attention_fp32(q, k, v, causal: bool = False, scale: float | None = None, window_left: int = -1, mask=None):
    """Reference tests/reference.py:26-54 (and :57-86 for the window): naive fp32 attention,
    GQA by repeat_interleave, bottom-right aligned causal mask.  ``mask``: additive natural-log
    bias broadcastable to [B, H, M, N], added to the scaled logits (the semantics of the
    reference's attn_fp16_fwd, csrc/include/attn_fp16_fwd.cuh:176-178)."""
    qf, kf, vf = (t.detach().cpu().float() for t in (q, k, v))
    kf, vf = _expand_kv(kf, vf, qf.shape[1])
    if scale is None:
        scale = 1.0 / math.sqrt(q.shape[-1])
    s = torch.einsum("bhmd,bhnd->bhmn", qf, kf) * scale
    if mask is not None:
        s = s + mask.detach().cpu().float()
    m_len, n_len = s.shape[-2], s.shape[-1]
    if window_left >= 0:
        row = torch.arange(m_len).view(-1, 1)
        col = torch.arange(n_len).view(1, -1)
        diff = (row + (n_len - m_len)) - col
        s = s.masked_fill(~((diff >= 0) & (diff < window_left)), float("-inf"))
    elif causal:
        keep = torch.ones(m_len, n_len, dtype=torch.bool).tril(n_len - m_len)
        s = s.masked_fill(~keep, float("-inf"))
    p = torch.softmax(s, dim=-1)
    return torch.einsum("bhmn,bhnd->bhmd", p, vf)


def attention_fp32_ragged(q, k, v, seqlens_q, seqlens_k, causal=False, scale=None):
    """Per-sequence loop over [:, :, :len] slices (the pattern of reference
    tests/reference.py:154-169); padded output rows are zero."""
    out = torch.zeros(q.shape, dtype=torch.float32)
    for b in range(q.shape[0]):
        mq, nk = int(seqlens_q[b]), int(seqlens_k[b])
        if mq and nk:
            out[b:b + 1, :, :mq] = attention_fp32(q[b:b + 1, :, :mq], k[b:b + 1, :, :nk], v[b:b + 1, :, :nk], causal, scale)
    return out


def varlen_smooth_k(k: torch.Tensor, cu_seqlens_k) -> torch.Tensor:
    """Reference superl8/ops.py:268-315 (`_varlen_smooth_k`): packed keys [total, H, D] minus the
    per-(head, channel) fp32 mean of each token's own sequence (`mean(dim=1)` over the sequence's
    tokens, as the reference forms it), rounded back to k's dtype."""
    kf = k.detach().cpu().float()
    bounds = [int(x) for x in cu_seqlens_k]
    parts = []
    for b in range(len(bounds) - 1):
        seg = kf[bounds[b]:bounds[b + 1]]
        if seg.shape[0]:
            parts.append((seg.unsqueeze(0) - seg.unsqueeze(0).mean(dim=1, keepdim=True)).squeeze(0).to(k.dtype))
    return torch.cat(parts, 0) if parts else kf.to(k.dtype)


def attn_int8_varlen(q, k, v, cu_seqlens_q, cu_seqlens_k, causal=False, scale=None, rule: str = "cuda"):
    """Reference superl8/ops.py:318-364 + csrc/include/attn_varlen_fwd.cuh:25-190 as a loop over
    sequences: smooth K per sequence, quantise rows, fold the scale, and run the int8 kernel
    mathematics (attn_int8_fwd above; bottom-right causal diagonal) on every sequence alone.
    q, k, v packed [total, H, D]; returns [total_q, Hq, D] in v's dtype."""
    if scale is None:
        scale = 1.0 / math.sqrt(q.shape[-1])
    k_s = varlen_smooth_k(k, cu_seqlens_k)
    q_i8, q_scale = quantize_rowwise(q.detach().cpu(), rule)
    k_i8, k_scale = quantize_rowwise(k_s, rule)
    q_scale = fold_scale(q_scale, scale)
    out = torch.zeros(q.shape, dtype=v.dtype)
    cq, ck = [int(x) for x in cu_seqlens_q], [int(x) for x in cu_seqlens_k]
    for b in range(len(cq) - 1):
        qs_, ks_ = slice(cq[b], cq[b + 1]), slice(ck[b], ck[b + 1])
        if cq[b + 1] == cq[b]:
            continue
        tr = lambda t: t.transpose(0, 1).unsqueeze(0).contiguous()      # [S, H, ...] -> [1, H, S, ...]
        o = attn_int8_fwd(tr(q_i8[qs_]), tr(q_scale[qs_]).squeeze(-1), tr(k_i8[ks_]), tr(k_scale[ks_]).squeeze(-1),
                          tr(v.detach().cpu()[ks_]), causal=causal)
        out[qs_] = o[0].transpose(0, 1)
    return out


def attention_fp32_varlen(q, k, v, cu_seqlens_q, cu_seqlens_k, causal=False, scale=None):
    """fp32 attention of every packed sequence on its own (the pattern of reference
    tests/reference.py:154-169)."""
    out = torch.zeros(q.shape, dtype=torch.float32)
    cq, ck = [int(x) for x in cu_seqlens_q], [int(x) for x in cu_seqlens_k]
    tr = lambda t: t.transpose(0, 1).unsqueeze(0)
    for b in range(len(cq) - 1):
        if cq[b + 1] > cq[b] and ck[b + 1] > ck[b]:
            o = attention_fp32(tr(q[cq[b]:cq[b + 1]]), tr(k[ck[b]:ck[b + 1]]), tr(v[ck[b]:ck[b + 1]]), causal, scale)
            out[cq[b]:cq[b + 1]] = o[0].transpose(0, 1)
    return out


def attention_lse_fp32(q, k, causal: bool = False, scale: float | None = None) -> torch.Tensor:
    """Natural-log row sums of the scaled, masked logits: what the forward saves for the
    backward, recomputed the way reference superl8/ops.py:49-58 does when it is missing."""
    qf, kf = q.detach().cpu().float(), k.detach().cpu().float()
    kf, _ = _expand_kv(kf, kf, qf.shape[1])
    if scale is None:
        scale = 1.0 / math.sqrt(q.shape[-1])
    s = torch.einsum("bhmd,bhnd->bhmn", qf, kf) * scale
    if causal:
        m_len, n_len = s.shape[-2], s.shape[-1]
        s = s.masked_fill(~torch.ones(m_len, n_len, dtype=torch.bool).tril(n_len - m_len), float("-inf"))
    return torch.logsumexp(s, dim=-1).float()


def attention_backward_fp32(q, k, v, out, d_out, causal: bool = False, scale: float | None = None, lse=None):
    """Exact FlashAttention-2 gradient in fp32: reference superl8/autograd.py:29-45, with the
    grouped-head sum the reference's kernel pair performs (csrc/include/attn_bwd.cuh:399-404).
    P = exp(S - lse) when ``lse`` is given (what the kernels do, attn_bwd.cuh:260), else softmax.
    Returns fp32 (dq [B,Hq,M,D], dk, dv [B,Hkv,N,D])."""
    qf, kf, vf, of, dof = (t.detach().cpu().float() for t in (q, k, v, out, d_out))
    Hq, Hkv = qf.shape[1], kf.shape[1]
    rep = Hq // Hkv
    kf, vf = _expand_kv(kf, vf, Hq)
    if scale is None:
        scale = 1.0 / math.sqrt(q.shape[-1])
    s = torch.einsum("bhmd,bhnd->bhmn", qf, kf) * scale
    if causal:
        m_len, n_len = s.shape[-2], s.shape[-1]
        s = s.masked_fill(~torch.ones(m_len, n_len, dtype=torch.bool).tril(n_len - m_len), float("-inf"))
    if lse is None:
        p = torch.softmax(s, dim=-1)
    else:
        p = torch.exp(s - lse.detach().cpu().float().unsqueeze(-1))
    p = torch.nan_to_num(p, nan=0.0)
    dv = torch.einsum("bhmn,bhmd->bhnd", p, dof)
    dp = torch.einsum("bhmd,bhnd->bhmn", dof, vf)
    drow = (dof * of).sum(dim=-1, keepdim=True)
    ds = p * (dp - drow)
    dq = torch.einsum("bhmn,bhnd->bhmd", ds, kf) * scale
    dk = torch.einsum("bhmn,bhmd->bhnd", ds, qf) * scale
    if rep > 1:
        B, _, N, D = dk.shape
        dk = dk.view(B, Hkv, rep, N, D).sum(dim=2)
        dv = dv.view(B, Hkv, rep, N, D).sum(dim=2)
    return dq, dk, dv


# --------------------------------------------------------------------------- kernel restatements

def int32_logits(q_i8: torch.Tensor, k_i8: torch.Tensor) -> torch.Tensor:
    """int32 Q.K^T (reference csrc/include/attn_int8_fwd.cuh:129-133: __dp4a chain).
    q [..., M, D], k [..., N, D] int8 -> int32 [..., M, N].  Exact: |acc| <= 127^2 * 256 < 2^31.
    For D <= 1024 every partial sum is an integer below 2^24, so an fp32 matrix product is exact
    in any summation order and is used for speed; larger D takes the integer product."""
    if q_i8.shape[-1] * 127 * 127 < (1 << 24):
        a, b = q_i8.detach().cpu().float(), k_i8.detach().cpu().float()
        return torch.matmul(a, b.transpose(-1, -2)).to(torch.int32)
    a = q_i8.detach().cpu().numpy().astype(np.int32)
    b = k_i8.detach().cpu().numpy().astype(np.int32)
    return torch.from_numpy(np.matmul(a, np.swapaxes(b, -1, -2)).astype(np.int32))


def attn_int8_fwd(q_i8, q_scale, k_i8, k_scale, v, causal=False, window_left=-1, want_lse=False):
    """Kernel mathematics of reference csrc/include/attn_int8_fwd.cuh:126-208, whole rows at
    once instead of 64-key tiles: s = float(acc) * q_scale[m] * k_scale[n]; masked -> -inf;
    p = exp2(s - rowmax); out = (p @ v) / l cast to v's dtype, 0 where l == 0;
    lse = m * ln2 + ln l.  q_scale [B,Hq,M], k_scale [B,Hkv,N]."""
    q_i8, k_i8, v = q_i8.detach().cpu(), k_i8.detach().cpu(), v.detach().cpu()
    qs, ks = q_scale.detach().cpu().float(), k_scale.detach().cpu().float()
    B, Hq, M, D = q_i8.shape
    Hkv, N = k_i8.shape[1], k_i8.shape[2]
    g = Hq // Hkv
    out = torch.zeros((B, Hq, M, D), dtype=v.dtype)
    lse = torch.full((B, Hq, M), float("-inf"), dtype=torch.float32)
    if N == 0 or M == 0:
        return (out, lse) if want_lse else out
    row = torch.arange(M).view(-1, 1)
    col = torch.arange(N).view(1, -1)
    pos = row + ((N - M) if causal else 0)
    valid = torch.ones(M, N, dtype=torch.bool)
    if causal:
        valid &= col <= pos
    if window_left >= 0:
        valid &= col > pos - window_left
    for b in range(B):
        for h in range(Hq):
            hk = h // g
            acc = int32_logits(q_i8[b, h], k_i8[b, hk]).float()
            s = acc * qs[b, h].view(-1, 1) * ks[b, hk].view(1, -1)
            s = torch.where(valid, s, torch.full_like(s, float("-inf")))
            m = s.amax(dim=-1, keepdim=True)
            m_safe = torch.where(torch.isinf(m), torch.zeros_like(m), m)
            p = torch.exp2(s - m_safe)
            l = p.sum(dim=-1, keepdim=True)
            o = p @ v[b, hk].float()
            inv = torch.where(l > 0, 1.0 / l, torch.zeros_like(l))
            out[b, h] = (o * inv).to(v.dtype)
            lse[b, h] = torch.where(l.squeeze(-1) > 0, m.squeeze(-1) * 0.6931471805599453 + torch.log(l.squeeze(-1)),
                                    torch.full_like(l.squeeze(-1), float("-inf")))
    return (out, lse) if want_lse else out


def attn_w8a8_fwd(q_i8, q_scale, k_i8, k_scale, v_i8, v_scale, causal=False, causal_diag=0, per_warp=True):
    """Reference csrc/include/attn_w8a8_fwd.cuh:93-222, tile by tile (64 keys): logits as in
    attn_int8_fwd; per tile m_new = max(m, tile max), P = exp2(s - m_new); p_scale =
    max(max(P) / 127, 2e-38) per row and tile, or per row and 32-key half (per_warp);
    P8 = rint(P / p_scale); O = O * exp2(m - m_new) + (P8 @ V8) * p_scale * v_scale; l from the
    unquantised P; out = O / l -> fp16.  q_scale [B,Hq,M], k_scale [B,Hkv,N], v_scale [B,Hkv,D]."""
    f32 = np.float32
    q_i8, k_i8, v_i8 = q_i8.detach().cpu(), k_i8.detach().cpu(), v_i8.detach().cpu()
    qs, ks = q_scale.detach().cpu().float().numpy(), k_scale.detach().cpu().float().numpy()
    B, Hq, M, D = q_i8.shape
    Hkv, N = k_i8.shape[1], k_i8.shape[2]
    vs = v_scale.detach().cpu().float().reshape(B, Hkv, D).numpy()
    g = Hq // Hkv
    out = torch.zeros((B, Hq, M, D), dtype=torch.float16)
    if M == 0 or N == 0:
        return out
    row = np.arange(M).reshape(-1, 1)
    col = np.arange(N).reshape(1, -1)
    valid = np.ones((M, N), dtype=bool)
    if causal:
        valid &= col <= row + causal_diag
    inv127 = f32(1.0) / f32(127.0)
    with np.errstate(over="ignore", invalid="ignore", divide="ignore"):
        for b in range(B):
            for h in range(Hq):
                hk = h // g
                acc = int32_logits(q_i8[b, h], k_i8[b, hk]).numpy().astype(f32)
                s = (acc * qs[b, h].reshape(-1, 1).astype(f32)) * ks[b, hk].reshape(1, -1).astype(f32)
                s = np.where(valid, s, -np.inf).astype(f32)
                v8 = v_i8[b, hk].numpy().astype(np.int32)
                m_i = np.full(M, -np.inf, dtype=f32)
                l_i = np.zeros(M, dtype=f32)
                o = np.zeros((M, D), dtype=f32)
                for n0 in range(0, N, 64):
                    st = s[:, n0:n0 + 64]
                    if st.shape[1] < 64:
                        st = np.concatenate([st, np.full((M, 64 - st.shape[1]), -np.inf, dtype=f32)], axis=1)
                    vt = np.zeros((64, D), dtype=np.int32)
                    vt[:min(64, N - n0)] = v8[n0:n0 + 64]
                    m_new = np.maximum(m_i, st.max(axis=1))
                    live = np.isfinite(m_new)
                    p = np.where(np.isfinite(st) & live[:, None], np.exp2(st - np.where(live, m_new, 0)[:, None]), 0).astype(f32)
                    rescale = np.where(np.isfinite(m_i) & live, np.exp2(m_i - np.where(live, m_new, 0)), 1).astype(f32)
                    o *= rescale[:, None]
                    l_i = (l_i * rescale + p.sum(axis=1, dtype=f32)).astype(f32)
                    m_i = np.maximum(m_i, m_new)
                    halves = ((0, 32), (32, 64)) if per_warp else ((0, 64),)
                    contrib = np.zeros((M, D), dtype=f32)
                    for lo, hi in halves:
                        pmax = p[:, lo:hi].max(axis=1)
                        p_scale = np.maximum(pmax * inv127, f32(2e-38)).astype(f32)
                        p8 = np.rint(p[:, lo:hi] * (f32(1.0) / p_scale)[:, None]).astype(np.int32)
                        contrib += (p8 @ vt[lo:hi]).astype(f32) * p_scale[:, None]
                    o += contrib * vs[b, hk].reshape(1, -1)
                inv = np.where(l_i > 0, f32(1.0) / np.where(l_i > 0, l_i, 1), 0).astype(f32)
                out[b, h] = torch.from_numpy((o * inv[:, None]).astype(np.float16))
    return out


def choose_n_splits_reference(n_len: int, bhq: int) -> int:
    """Reference csrc/kernel/attn_decode.cu:33-53."""
    if n_len <= 0 or bhq <= 0:
        return 1
    s_occ = (2048 + bhq - 1) // bhq
    s_lo = (n_len + 255) // 256
    s_hi = max(1, (n_len + 47) // 48)
    return max(1, min(min(max(s_occ, s_lo), s_hi), 256))


def quantize_v_perchannel(v: torch.Tensor):
    """Reference superl8/quant/core.py:98-110: symmetric int8 per CHANNEL of V (scale over the
    key axis), scale = amax / 127 (0 -> 1).  Returns (v_i8 [..., N, D], scale fp32 [..., 1, D])."""
    vf = v.detach().cpu().float()
    scale = vf.abs().amax(dim=-2, keepdim=True) / Q_MAX
    safe = torch.where(scale == 0, torch.ones_like(scale), scale)
    return torch.round(vf / safe).clamp_(-Q_MAX, Q_MAX).to(torch.int8), safe


def attn_int8_decode(q_i8, q_scale, k_i8, k_scale, v, n_splits: int = 1, context_lens=None, v_scale=None):
    """Reference csrc/include/attn_decode.cuh:68-131 (split) and :442-465 (combine): split s
    owns keys [s*per, min(len, (s+1)*per)), per = ceil(N / n_splits); partial (o, m, l) in
    the exp2 domain; merge o = sum o_s 2^(m_s - gm) / sum l_s 2^(m_s - gm) -> fp16.
    q_i8 [B,Hq,1,D], q_scale [B,Hq(,1)], k_i8 [B,Hkv,N,D], k_scale [B,Hkv,N], v fp16 -- or, with
    ``v_scale`` [B,Hkv,D], the int8-V cache of attn_decode.cuh:141-224: o accumulates
    p * float(v_i8) and the per-channel scale multiplies the partial."""
    q_i8, k_i8, v = q_i8.detach().cpu(), k_i8.detach().cpu(), v.detach().cpu()
    qs = q_scale.detach().cpu().float().reshape(q_i8.shape[0], q_i8.shape[1])
    ks = k_scale.detach().cpu().float()
    B, Hq, _, D = q_i8.shape
    Hkv, N = k_i8.shape[1], k_i8.shape[2]
    g = Hq // Hkv
    out = torch.zeros((B, Hq, 1, D), dtype=torch.float16)
    if N == 0:
        return out
    per = (N + n_splits - 1) // n_splits
    for b in range(B):
        n_b = N if context_lens is None else min(int(context_lens[b]), N)
        for h in range(Hq):
            hk = h // g
            acc = int32_logits(q_i8[b, h], k_i8[b, hk, :n_b]).float().view(-1)
            s = acc * qs[b, h] * ks[b, hk, :n_b]
            ms, ls, os_ = [], [], []
            for sp in range(n_splits):
                n0, n1 = sp * per, min(n_b, (sp + 1) * per)
                if n1 <= n0:
                    continue
                m = s[n0:n1].max()
                p = torch.exp2(s[n0:n1] - m)
                ms.append(m)
                ls.append(p.sum())
                o_s = p @ v[b, hk, n0:n1].float()
                os_.append(o_s if v_scale is None else o_s * v_scale.detach().cpu().float().reshape(B, Hkv, D)[b, hk])
            if not ms:
                continue
            gm = torch.stack(ms).max()
            w = torch.exp2(torch.stack(ms) - gm)
            denom = (torch.stack(ls) * w).sum()
            o = (torch.stack(os_) * w.view(-1, 1)).sum(dim=0)
            out[b, h, 0] = (o / denom if denom > 0 else torch.zeros_like(o)).to(torch.float16)
    return out


# --------------------------------------------------------------------------- gates (reference tests/tolerances.py)

def sqnr_db(out, ref) -> float:
    ref_f, out_f = ref.detach().cpu().float(), out.detach().cpu().float()
    noise = (out_f - ref_f).pow(2).mean()
    signal = ref_f.pow(2).mean()
    if noise == 0:
        return float("inf")
    return (10.0 * torch.log10(signal / noise)).item()


def cos_sim(out, ref) -> float:
    a, b = out.detach().cpu().float().flatten(), ref.detach().cpu().float().flatten()
    return torch.nn.functional.cosine_similarity(a, b, dim=0).item()


def rel_l1(out, ref) -> float:
    ref_f = ref.detach().cpu().float()
    return ((out.detach().cpu().float() - ref_f).abs().sum() / ref_f.abs().sum().clamp_min(1e-12)).item()


def assert_int8_quality(out, ref, *, min_cos=0.999, max_rel_l1=0.02, min_sqnr_db=20.0, what="int8 output"):
    """The reference's one int8 gate (tests/tolerances.py:74-88)."""
    assert torch.isfinite(out.detach().cpu().float()).all(), f"{what} contains NaN/Inf"
    c, l1, s = cos_sim(out, ref), rel_l1(out, ref), sqnr_db(out, ref)
    assert c >= min_cos, f"{what}: cos-sim {c:.6f} < {min_cos}"
    assert l1 <= max_rel_l1, f"{what}: rel-L1 {l1:.4f} > {max_rel_l1}"
    assert s >= min_sqnr_db, f"{what}: SQNR {s:.1f} dB < {min_sqnr_db} dB"


# --------------------------------------------------------------------------- synthetic inputs

def make_qkv(seed: int, Hq: int, Hkv: int, S: int, D: int, Sk: int | None = None, dtype=torch.float16):
    """One batch element: Q [Hq,S,D], K, V [Hkv,Sk,D] drawn in that order from a CPU
    generator seeded with ``seed``, ~N(0,1), cast to ``dtype``."""
    g = torch.Generator().manual_seed(seed)
    Sk = S if Sk is None else Sk
    q = torch.randn(Hq, S, D, generator=g).to(dtype)
    k = torch.randn(Hkv, Sk, D, generator=g).to(dtype)
    v = torch.randn(Hkv, Sk, D, generator=g).to(dtype)
    return q, k, v


def make_batch(cfg: int, B: int, Hq: int, Hkv: int, S: int, D: int, Sk: int | None = None, dtype=torch.float16,
               first_b: int = 0):
    """Batch elements first_b .. first_b + B - 1 of a configuration: seed = 1000 * cfg + b."""
    qs, ks, vs = zip(*(make_qkv(1000 * cfg + first_b + b, Hq, Hkv, S, D, Sk, dtype) for b in range(B)))
    return torch.stack(qs), torch.stack(ks), torch.stack(vs)


def outlier_channels(H: int, D: int, seed: int, frac: float = 0.01) -> torch.Tensor:
    """Mask [H, D] of the ceil(frac * H * D) channels that get scaled x20."""
    n = math.ceil(frac * H * D)
    idx = torch.randperm(H * D, generator=torch.Generator().manual_seed(seed))[:n]
    mask = torch.zeros(H * D, dtype=torch.bool)
    mask[idx] = True
    return mask.view(H, D)
