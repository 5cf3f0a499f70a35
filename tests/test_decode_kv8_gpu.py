"""int8 K / int8 V cached decode (per-channel V scales) through the C ABI: the V quantiser
bit-exact against the restated reference, the decode against the reference's own int8-V kernels
on the same inputs and against the oracle."""

import pytest
import torch

import superl8_b200 as s8
from gpu_helpers import ref_attn_int8_decode_kv8, ref_lib
from oracle import oracle
from superl8_b200 import _C, quant

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("shape,dtype", [((2, 2, 300, 64), torch.float16), ((1, 3, 2500, 128), torch.bfloat16),
                                         ((1, 1, 1, 32), torch.float16), ((2, 1, 1024, 256), torch.float16)])
def test_v_perchannel_quantiser_bit_exact(device, shape, dtype):
    g = torch.Generator().manual_seed(shape[2])
    v = (torch.randn(*shape, generator=g) * 1.3).to(dtype)
    if shape[2] > 20:
        v[0, 0, :, 3] = 0
        v[-1, -1, 7, 1] = 200.0
    v_i8, v_scale = quant.quantize_v_perchannel(v.to(device))
    qo, so = oracle.quantize_v_perchannel(v)
    assert v_scale.shape == so.shape and torch.equal(v_scale.cpu(), so)
    assert torch.equal(v_i8.cpu(), qo)


CASES = [  # B, Hq, Hkv, N, D
    (2, 8, 2, 777, 128), (1, 16, 1, 4100, 64), (3, 4, 4, 65, 32), (1, 8, 8, 1500, 256), (2, 64, 8, 3000, 128),
]


@pytest.mark.parametrize("case", CASES)
def test_decode_kv8_matches_reference_kernel_and_oracle(device, case):
    B, Hq, Hkv, N, D = case
    g = torch.Generator().manual_seed(N + D)
    q = torch.randn(B, Hq, 1, D, generator=g).half()
    k = (torch.randn(B, Hkv, N, D, generator=g) + 0.3).half()
    v = torch.randn(B, Hkv, N, D, generator=g).half()
    k_i8, k_scale, v_i8, v_scale = s8.quantize_kv_cache(k.to(device), v.to(device))
    assert k_i8.dtype == torch.int8 and v_i8.dtype == torch.int8 and v_scale.shape == (B, Hkv, D)
    scale = D ** -0.5
    q_i8, q_scale = oracle.quantize_rowwise(q, "cuda")
    q_scale = oracle.fold_scale(q_scale, scale).reshape(B, Hq, 1).contiguous()
    outs = {}
    for ns in (1, 3, -1):
        outs[ns] = _C.attn_int8_decode_kv8(q_i8.to(device), q_scale.to(device), k_i8, k_scale, v_i8, v_scale, ns)
        assert outs[ns].shape == (B, Hq, 1, D) and outs[ns].dtype == torch.float16
    assert _C.device_status() == 0
    ref_o = oracle.attn_int8_decode(q_i8, q_scale, k_i8, k_scale, v_i8, n_splits=3, v_scale=v_scale)
    for ns, out in outs.items():
        assert oracle.cos_sim(out, ref_o) >= 0.99999 and oracle.rel_l1(out, ref_o) <= 3e-3, ns
    if ref_lib() is not None:
        ref_k = ref_attn_int8_decode_kv8(q_i8.to(device), q_scale.to(device), k_i8, k_scale, v_i8, v_scale, 3)
        assert oracle.cos_sim(outs[3], ref_k) >= 0.99999 and oracle.rel_l1(outs[3], ref_k) <= 3e-3
    # public wrapper = same thing with the library's own Q quantiser; and the int8 cache stays
    # within the reference's int8 gate of full-precision attention over the same K/V
    pub = s8.attn_decode_cached(q.to(device), k_i8, k_scale, v_i8, v_scale)
    assert oracle.cos_sim(pub, outs[-1]) >= 0.99999
    oracle.assert_int8_quality(pub, oracle.attention_fp32(q, k, v))


def test_decode_kv8_context_lens_and_errors(device):
    B, Hq, Hkv, N, D = 3, 8, 2, 600, 128
    g = torch.Generator().manual_seed(5)
    q = torch.randn(B, Hq, 1, D, generator=g).half().to(device)
    k = torch.randn(B, Hkv, N, D, generator=g).half().to(device)
    v = torch.randn(B, Hkv, N, D, generator=g).half().to(device)
    lens = torch.tensor([600, 1, 333], dtype=torch.int32, device=device)
    k_i8, k_scale, v_i8, v_scale = s8.quantize_kv_cache(k, v)
    out = s8.attn_decode_cached(q, k_i8, k_scale, v_i8, v_scale, context_lens=lens)
    for b in range(B):
        n = int(lens[b])
        one = s8.attn_decode_cached(q[b:b + 1], k_i8[b:b + 1, :, :n].contiguous(), k_scale[b:b + 1, :, :n].contiguous(),
                                    v_i8[b:b + 1, :, :n].contiguous(), v_scale[b:b + 1])
        assert oracle.cos_sim(out[b:b + 1], one) >= 0.99999
    with pytest.raises(RuntimeError, match="per-token"):
        s8.attn_decode_cached(q, k_i8, k_scale, v_i8, k_scale)
    with pytest.raises(RuntimeError, match="int8"):
        _C.attn_int8_decode_kv8(k_i8[:, :, :1], k_scale[:, :, :1], k_i8, k_scale, v, v_scale, -1)
    with pytest.raises(NotImplementedError):
        s8.quantize_kv_cache(k, v, v_quant="per_token")


def test_rotated_cache_keeps_the_logits_and_tightens_an_outlier_channel(device):
    """rotate=True on both sides (cache built once, every query rotated the same way) leaves q.k
    unchanged (reference superl8/ops.py:671-727 with superl8/quant/rotation.py): decode against the
    rotated int8 cache meets the int8-V bar, and with an outlier channel in K it is closer to fp32
    attention than the unrotated cache."""
    gen = torch.Generator().manual_seed(81)
    B, Hq, Hkv, N, D = 2, 8, 2, 1500, 128
    q = torch.randn(B, Hq, 1, D, generator=gen).half()
    k = torch.randn(B, Hkv, N, D, generator=gen).half()
    k[..., 9] *= 25.0
    v = torch.randn(B, Hkv, N, D, generator=gen).half()
    ref = oracle.attention_fp32(q, k, v)
    errs = {}
    for rotate in (False, True):
        k8, ks, v8, vs = s8.quantize_kv_cache(k.to(device), v.to(device), rotate=rotate)
        out = s8.attn_decode_cached(q.to(device), k8, ks, v8, vs, rotate=rotate)
        errs[rotate] = oracle.rel_l1(out, ref)
        assert torch.isfinite(out.float()).all()
    assert errs[True] <= 0.03 and errs[True] < errs[False]
    # the one-pass cache quantiser equals its pieces: smooth, rotate, plain quantiser
    k8, ks, _, _ = s8.quantize_kv_cache(k.to(device), v.to(device), rotate=True)
    k_s = quant.smooth_quantize_k(k.to(device), quant.k_mean(k.to(device)), want_smoothed=True)[2]
    r8, rs = quant.quantize_int8_rowwise(quant.rotate_last(k_s))
    assert torch.equal(k8, r8) and torch.equal(ks, rs.squeeze(-1))
