"""GPU parity of the split-KV decode (int8 K + per-token scales, fp16 V), through the C ABI."""

import pytest
import torch

import superl8_b200 as s8
from gpu_helpers import quantized_inputs, ref_decode, ref_lib
from oracle import oracle
from superl8_b200 import _C

pytestmark = pytest.mark.gpu

# (B, Hq, Hkv, N, D): MHA / GQA / MQA, ragged N, every head dim the reference decodes
SHAPES = [(2, 8, 8, 512, 64), (2, 8, 2, 777, 128), (1, 16, 1, 2000, 64), (3, 4, 4, 100, 32), (1, 8, 2, 1030, 256),
          (2, 32, 2, 300, 128), (1, 40, 2, 129, 128), (4, 64, 8, 4096, 128), (1, 2, 1, 1, 64), (1, 8, 8, 63, 128)]


def run(d, ns=-1, lens=None):
    dev = d["dev"]
    return _C.attn_int8_decode(dev["q_i8"], dev["q_scale"], dev["k_i8"], dev["k_scale"], dev["v"], ns,
                               context_lens=lens)


@pytest.mark.parametrize("B,Hq,Hkv,N,D", SHAPES)
def test_decode_vs_oracle_and_reference_kernel(B, Hq, Hkv, N, D, device):
    d = quantized_inputs(50 + D, B, Hq, Hkv, 1, D, N=N)
    out = run(d)
    assert out.shape == (B, Hq, 1, D) and out.dtype == torch.float16
    assert _C.device_status() == 0
    oracle.assert_int8_quality(out, oracle.attention_fp32(d["q"], d["k"], d["v"]), what="decode vs fp32 oracle")
    rest = oracle.attn_int8_decode(d["q_i8"], d["q_scale"], d["k_i8"], d["k_scale"], d["v"], n_splits=1)
    assert oracle.cos_sim(out, rest) >= 0.99999 and oracle.rel_l1(out, rest) <= 3e-3
    if ref_lib() is not None:
        dev = d["dev"]
        r = ref_decode(dev["q_i8"], dev["q_scale"], dev["k_i8"], dev["k_scale"], dev["v"],
                       oracle.choose_n_splits_reference(N, B * Hq))
        assert oracle.cos_sim(out, r) >= 0.99999 and oracle.rel_l1(out, r) <= 3e-3
    assert torch.equal(out, run(d))                           # bitwise repeatable


def test_split_count_invariance_and_rejection(device):
    d = quantized_inputs(61, 1, 8, 2, 1, 128, N=5000)
    base = run(d, 1)
    for ns in (2, 3, 7, 16, 64, 256):
        assert oracle.cos_sim(run(d, ns), base) >= 0.99999, ns
    for bad in (0, 257):
        with pytest.raises(RuntimeError, match="num_splits"):
            run(d, bad)
    dev = d["dev"]
    with pytest.raises(RuntimeError, match="float16"):
        _C.attn_int8_decode(dev["q_i8"], dev["q_scale"], dev["k_i8"], dev["k_scale"], dev["v"].bfloat16(), -1)


def test_decode_equals_prefill_kernel_at_m1(device):
    d = quantized_inputs(62, 2, 8, 2, 1, 128, N=640)
    dev = d["dev"]
    pre = _C.attn_int8_fwd(dev["q_i8"], dev["q_scale"], dev["k_i8"], dev["k_scale"], dev["v"], False, -1)
    assert oracle.cos_sim(run(d), pre) >= 0.999


def test_ragged_context_lens(device):
    B, Hq, Hkv, N, D = 5, 16, 2, 3000, 128
    d = quantized_inputs(63, B, Hq, Hkv, 1, D, N=N)
    lens = torch.tensor([3000, 1, 64, 1025, 0], dtype=torch.int32)
    out = run(d, -1, lens.to(device))
    out8 = run(d, 8, lens.to(device))
    rest = oracle.attn_int8_decode(d["q_i8"], d["q_scale"], d["k_i8"], d["k_scale"], d["v"], n_splits=1,
                                   context_lens=lens)
    assert oracle.cos_sim(out, rest) >= 0.99999 and oracle.cos_sim(out8, rest) >= 0.99999
    assert float(out[4].abs().max()) == 0.0                   # empty sequence -> zeros


def test_empty_cache_gives_zeros(device):
    q = torch.zeros(2, 4, 1, 64, dtype=torch.int8, device=device)
    qs = torch.ones(2, 4, 1, device=device)
    k = torch.zeros(2, 2, 0, 64, dtype=torch.int8, device=device)
    ks = torch.zeros(2, 2, 0, device=device)
    v = torch.zeros(2, 2, 0, 64, dtype=torch.float16, device=device)
    out = _C.attn_int8_decode(q, qs, k, ks, v, -1)
    assert out.shape == (2, 4, 1, 64) and float(out.abs().max()) == 0.0


def test_python_entry_points(device):
    q, k, v = oracle.make_batch(64, 2, 8, 2, 1, 128, Sk=900)
    ref = oracle.attention_fp32(q, k, v)
    out = s8.attn_int8_decode(q.to(device), k.to(device), v.to(device))
    oracle.assert_int8_quality(out, ref)
    assert torch.equal(out, s8.attn_decode(q.to(device), k.to(device), v.to(device)))
    _qi, _qs, k_i8, k_scale, _ = s8.quantize_qk(q.to(device), k.to(device))
    out2 = s8.attn_decode_int8_cache(q.to(device), k_i8, k_scale.squeeze(-1).contiguous(), v.to(device))
    assert torch.equal(out, out2)


def test_long_context_property(device):
    # BASELINE-size sequence (N = 32768): V = const c per channel -> output = c exactly-ish
    B, Hq, Hkv, N, D = 1, 64, 8, 32768, 128
    g = torch.Generator().manual_seed(7)
    q_i8 = torch.randint(-127, 128, (B, Hq, 1, D), generator=g, dtype=torch.int8).to(device)
    k_i8 = torch.randint(-127, 128, (B, Hkv, N, D), generator=g, dtype=torch.int8).to(device)
    qs = torch.full((B, Hq, 1), 1e-3, device=device)
    ks = torch.full((B, Hkv, N), 1e-2, device=device)
    c = torch.linspace(-2, 2, D).half()
    v = c.view(1, 1, 1, D).expand(B, Hkv, N, D).contiguous().to(device)
    out = _C.attn_int8_decode(q_i8, qs, k_i8, ks, v, -1)
    assert torch.allclose(out.float().cpu(), c.float().view(1, 1, 1, D).expand(B, Hq, 1, D), atol=4e-3)
