"""Packed variable-length prefill (token-major [total, H, D] + cu_seqlens) through the C ABI:
the K prologue against the restated reference, the attention against the reference's own packed
kernel on the same int8 inputs, against the per-sequence oracle, and against the dense op."""

import pytest
import torch

import superl8_b200 as s8
from gpu_helpers import ref_attn_int8_varlen, ref_lib
from oracle import oracle
from superl8_b200 import _C, _lib, quant

pytestmark = pytest.mark.gpu
TC, MMA = _lib.SL8_BACKEND_TCGEN05, _lib.SL8_BACKEND_MMA


def _packed(lens_q, lens_k, Hq, Hkv, D, seed):
    g = torch.Generator().manual_seed(seed)
    cu_q = torch.tensor([0] + torch.tensor(lens_q).cumsum(0).tolist(), dtype=torch.int32)
    cu_k = torch.tensor([0] + torch.tensor(lens_k).cumsum(0).tolist(), dtype=torch.int32)
    q = torch.randn(int(cu_q[-1]), Hq, D, generator=g).half()
    k = (torch.randn(int(cu_k[-1]), Hkv, D, generator=g) + 0.2).half()
    v = torch.randn(int(cu_k[-1]), Hkv, D, generator=g).half()
    return q, k, v, cu_q, cu_k


def test_packed_k_prologue(device):
    q, k, v, cu_q, cu_k = _packed([5], [37, 5, 0, 300, 64], 2, 2, 64, 1)
    B = cu_k.numel() - 1
    mean_o = torch.zeros(B, 2, 64)
    for b in range(B):
        seg = k[int(cu_k[b]):int(cu_k[b + 1])].float()
        if seg.shape[0]:
            mean_o[b] = seg.unsqueeze(0).mean(dim=1)[0]
    k_i8, k_scale, mean, _ = quant.varlen_smooth_quantize_k(k.to(device), cu_k.to(device))
    assert torch.allclose(mean.cpu(), mean_o, rtol=1e-5, atol=1e-6)
    # given the SAME means: smoothed keys, codes and scales are bit-exact
    k_i8, k_scale, _, k_s = quant.varlen_smooth_quantize_k(k.to(device), cu_k.to(device), want_smoothed=True,
                                                           k_mean_override=mean_o)
    ks_o = oracle.varlen_smooth_k(k, cu_k)
    qo, so = oracle.quantize_rowwise(ks_o, rule="cuda")
    assert torch.equal(k_s.cpu(), ks_o)
    assert torch.equal(k_i8.cpu(), qo) and torch.equal(k_scale.cpu(), so)


CASES = [  # lens_q, lens_k, Hq, Hkv, D
    ([100, 7, 300, 64], [100, 7, 300, 64], 4, 2, 64),
    ([129, 1, 200], [129, 1, 200], 8, 2, 128),
    ([40, 130], [90, 300], 4, 1, 128),          # queries are the tail of a cached prefix
    ([65, 33, 0, 128], [65, 33, 0, 128], 2, 2, 32),
]


@pytest.mark.parametrize("case", CASES)
@pytest.mark.parametrize("causal", [False, True])
def test_varlen_matches_reference_kernel_and_oracle(device, case, causal):
    lens_q, lens_k, Hq, Hkv, D = case
    q, k, v, cu_q, cu_k = _packed(lens_q, lens_k, Hq, Hkv, D, 100 + D + len(lens_q))
    scale = D ** -0.5
    # same int8 inputs for everybody (oracle quantiser, CUDA rule)
    q_i8, q_scale = oracle.quantize_rowwise(q, "cuda")
    q_scale = oracle.fold_scale(q_scale, scale).squeeze(-1).contiguous()
    k_i8, k_scale = oracle.quantize_rowwise(oracle.varlen_smooth_k(k, cu_k), "cuda")
    k_scale = k_scale.squeeze(-1).contiguous()
    dv = lambda t: t.to(device)
    backends = [MMA] if D == 32 else [TC, MMA]
    outs = []
    for be in backends:
        out = _C.attn_int8_varlen(dv(q_i8), dv(q_scale), dv(k_i8), dv(k_scale), dv(v), dv(cu_q), dv(cu_k), max(lens_q),
                                  causal, backend=be)
        assert out.shape == q.shape and out.dtype == torch.float16
        outs.append(out)
        assert torch.equal(out, _C.attn_int8_varlen(dv(q_i8), dv(q_scale), dv(k_i8), dv(k_scale), dv(v), dv(cu_q),
                                                    dv(cu_k), max(lens_q), causal, backend=be))
    assert _C.device_status() == 0
    ref_o = oracle.attn_int8_varlen(q, k, v, cu_q, cu_k, causal=causal, scale=scale)
    for out in outs:
        assert oracle.cos_sim(out, ref_o) >= 0.99999 and oracle.rel_l1(out, ref_o) <= 3e-3
    if ref_lib() is not None:
        ref_k = ref_attn_int8_varlen(dv(q_i8), dv(q_scale), dv(k_i8), dv(k_scale), dv(v), dv(cu_q), dv(cu_k), max(lens_q),
                                     causal)
        for out in outs:
            assert oracle.cos_sim(out, ref_k) >= 0.99999 and oracle.rel_l1(out, ref_k) <= 3e-3
    # the reference's one gate against fp32 attention of every sequence alone
    oracle.assert_int8_quality(outs[0], oracle.attention_fp32_varlen(q, k, v, cu_q, cu_k, causal, scale))


def test_public_varlen_equals_dense_per_sequence(device):
    lens = [150, 64, 257]
    q, k, v, cu_q, cu_k = _packed(lens, lens, 4, 2, 128, 9)
    out = s8.attn_int8_varlen(q.to(device), k.to(device), v.to(device), cu_q.to(device), cu_k.to(device), max(lens),
                              max(lens), causal=True)
    for b, n in enumerate(lens):
        sl = slice(int(cu_q[b]), int(cu_q[b + 1]))
        tr = lambda t: t[sl].transpose(0, 1).unsqueeze(0).contiguous().to(device)
        dense = s8.attn_int8_fwd(tr(q), tr(k), tr(v), causal=True, internal_accuracy_gate=False)
        assert oracle.cos_sim(out[sl], dense[0].transpose(0, 1)) >= 0.9999


def test_varlen_errors(device):
    q, k, v, cu_q, cu_k = _packed([16], [16], 2, 2, 64, 3)
    q_i8, qs = oracle.quantize_rowwise(q)
    a = [q_i8.to(device), qs.squeeze(-1).contiguous().to(device), q_i8.to(device), qs.squeeze(-1).contiguous().to(device),
         v.to(device), cu_q.to(device), cu_k.to(device), 16]
    with pytest.raises(RuntimeError, match="int32"):
        _C.attn_int8_varlen(*a[:5], cu_q.long().to(device), a[6], 16)
    with pytest.raises(RuntimeError, match="head dim"):
        x = torch.zeros(16, 2, 96, dtype=torch.int8, device=device)
        _C.attn_int8_varlen(x, a[1], x, a[3], torch.zeros(16, 2, 96, dtype=torch.float16, device=device), a[5], a[6], 16)
    with pytest.raises(RuntimeError, match="cu_seqlens mismatch"):
        _C.attn_int8_varlen(*a[:6], torch.zeros(3, dtype=torch.int32, device=device), 16)
