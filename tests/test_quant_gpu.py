"""GPU parity of the quantiser and the Q/K prologues, through the C ABI.
Bit-exact targets: the oracle's CUDA scale rule, the reference's own kernel (oracle/_ref)
and the CUDA-eager torch formula the reference tests use (tests/test_quant_rowwise.py:42-52)."""

import numpy as np
import pytest
import torch

import superl8_b200 as s8
from conftest import GOLDEN, from_bits
from gpu_helpers import ref_lib, ref_quantize
from oracle import oracle
from superl8_b200 import _C, _lib, quant

pytestmark = pytest.mark.gpu

SHAPES = [(37, 128, torch.float16), (50, 64, torch.float16), (33, 128, torch.bfloat16), (21, 72, torch.float32),
          (19, 33, torch.float16), (17, 256, torch.float16), (1000, 80, torch.float16), (64, 1024, torch.bfloat16),
          (8, 4096, torch.float16), (3, 20000, torch.float16), (301, 32, torch.float16), (5, 7, torch.float32)]


def eager_cuda_oracle(x):
    """The reference tests' independent oracle, run by torch on the device."""
    scale = x.float().abs().amax(dim=-1, keepdim=True) / 127.0
    safe = torch.where(scale == 0, torch.ones_like(scale), scale)
    return torch.round(x.float() / safe).clamp_(-127.0, 127.0).to(torch.int8), safe.squeeze(-1)


@pytest.mark.parametrize("M,K,dtype", SHAPES)
def test_rowwise_bit_exact(M, K, dtype, device):
    x = (torch.randn(M, K, generator=torch.Generator().manual_seed(M * 7 + K)) * 2.5).to(dtype)
    x[0] = 0
    if M > 2:
        x[1, K // 2] = 900.0
        x[2] = x[2] * 1e-3
    q, s = s8.quantize_i8_rowwise(x.to(device))
    qo, so = oracle.quantize_rowwise(x, rule="cuda")
    assert torch.equal(s.cpu(), so.squeeze(-1))
    assert torch.equal(q.cpu(), qo)
    qe, se = eager_cuda_oracle(x.to(device))
    assert torch.equal(s, se) and torch.equal(q, qe)
    assert int(q.min()) >= -127 and float(s[0]) == 1.0 and int(q[0].abs().max()) == 0
    if ref_lib() is not None:
        qr, sr = ref_quantize(x.to(device))
        assert torch.equal(q, qr) and torch.equal(s, sr)
    q2, s2 = s8.quantize_i8_rowwise(x.to(device))
    assert torch.equal(q, q2) and torch.equal(s, s2)


def test_rowwise_golden_inputs(device):
    g = np.load(GOLDEN / "quant_rowwise.npz")
    for n in sorted({k.split("__")[0] for k in g.files}):
        x = from_bits(g[f"{n}__x"], str(g[f"{n}__dtype"]))
        q, s = s8.quantize_i8_rowwise(x.to(device))
        qo, so = oracle.quantize_rowwise(x, rule="cuda")
        assert torch.equal(q.cpu(), qo) and torch.equal(s.cpu(), so.squeeze(-1)), n
        # against the reference's CPU branch the scale may be 1 ulp off (amax/127 vs amax*(1/127))
        assert np.abs(q.cpu().numpy().astype(int) - g[f"{n}__q"].astype(int)).max() <= 1


def test_rowwise_empty_and_nd(device):
    q, s = s8.quantize_i8_rowwise(torch.empty(0, 128, dtype=torch.float16, device=device))
    assert q.shape == (0, 128) and s.shape == (0,)
    x = torch.randn(2, 3, 5, 64, device=device).half()
    q, s = s8.quantize_int8_rowwise(x)
    assert q.shape == x.shape and s.shape == (2, 3, 5, 1)
    with pytest.raises(RuntimeError, match="float16"):
        s8.quantize_i8_rowwise(torch.zeros(4, 8, dtype=torch.float64, device=device))


def test_full_size_config_rows_against_eager(device):
    # cfg2 Q: 1 x 32 x 4096 x 128 (131072 rows), checked against the CUDA-eager formula
    x = torch.randn(32 * 4096, 128, device=device).half()
    q, s = s8.quantize_i8_rowwise(x)
    qe, se = eager_cuda_oracle(x)
    assert torch.equal(q, qe) and torch.equal(s, se)
    # round trip property: |x - q*s| <= s/2 (+ fp rounding)
    err = (x.float() - q.float() * s[:, None]).abs()
    assert bool((err <= s[:, None] * 0.5001).all())
    assert int(q.abs().amax(dim=-1).min()) == 127


@pytest.mark.parametrize("D,dtype", [(128, torch.float16), (64, torch.float16), (256, torch.bfloat16), (80, torch.float16)])
def test_q_prologue_fold_and_gate(D, dtype, device):
    g = torch.Generator().manual_seed(D)
    qf = torch.randn(2, 3, 70, D, generator=g).to(dtype)
    sc = 0.11
    q_i8, q_scale, flag = quant.quantize_q(qf.to(device), sc, want_gate=True)
    qo, so = oracle.quantize_rowwise(qf, rule="cuda")
    assert torch.equal(q_i8.cpu(), qo)
    assert torch.equal(q_scale.cpu(), oracle.fold_scale(so, sc))
    assert bool(flag.item()) == oracle.detect_q_outlier_domination(qf)
    spiked = qf.clone()
    spiked[1, 2, 33, D // 3] = 80.0
    assert s8.detect_q_outlier_domination(spiked.to(device)) is True
    assert oracle.detect_q_outlier_domination(spiked) is True


def test_gate_on_golden_cases(device):
    g = np.load(GOLDEN / "outlier_gate.npz")
    for n in ("clean", "spike", "chan20", "d64", "near"):
        q = from_bits(g[f"{n}__q"], "float16")
        assert s8.detect_q_outlier_domination(q.to(device)) == bool(g[f"{n}__flag"]), n
    near = from_bits(g["near__q"], "float16")
    for r, want in enumerate([False, True, False, False]):
        assert s8.detect_q_outlier_domination(near[:, :, r:r + 1].contiguous().to(device)) == want


@pytest.mark.parametrize("shape,dtype", [((2, 2, 300, 64), torch.float16), ((1, 1, 2500, 64), torch.float16),
                                         ((1, 2, 130, 128), torch.bfloat16), ((1, 3, 1025, 256), torch.float16)])
def test_k_prologue(shape, dtype, device):
    g = torch.Generator().manual_seed(shape[2])
    k = (torch.randn(*shape, generator=g) * 1.5 + 0.4).to(dtype)
    mean_o = oracle.k_mean_fp32(k)
    mean = quant.k_mean(k.to(device))
    assert torch.equal(mean, quant.k_mean(k.to(device)))           # fixed summation order
    rel = ((mean.cpu() - mean_o).abs() / mean_o.abs().clamp_min(1e-3)).max().item()
    assert rel <= 1e-5, rel                                          # reference's own bar is 1e-6 on sums of 1k rows
    # given the SAME mean the smoothed values, codes and scales are bit-exact
    k_i8, k_scale, k_s = quant.smooth_quantize_k(k.to(device), mean_o.to(device), want_smoothed=True)
    ks_o, _ = oracle.smooth_k(k, mean_o)
    qo, so = oracle.quantize_rowwise(ks_o, rule="cuda")
    assert torch.equal(k_s.cpu(), ks_o)
    assert torch.equal(k_i8.cpu(), qo) and torch.equal(k_scale.cpu(), so)
    # fused mean: codes may differ where a 1-ulp mean change flips a rounding; must stay rare and +-1
    k_i8_f, _ks_f, _ = quant.smooth_quantize_k(k.to(device), mean)
    diff = (k_i8_f.cpu().int() - qo.int()).abs()
    assert int(diff.max()) <= 1 and float((diff > 0).float().mean()) < 2e-3


def test_k_mean_with_seqlens(device):
    k = torch.randn(3, 2, 200, 64).half()
    lens = torch.tensor([200, 57, 1], dtype=torch.int32)
    mean = quant.k_mean(k.to(device), lens.to(device)).cpu()
    for b in range(3):
        ref = oracle.k_mean_fp32(k[b:b + 1, :, :int(lens[b])])
        assert torch.allclose(mean[b:b + 1], ref, rtol=1e-5, atol=1e-6)


def test_quantize_qk_matches_oracle_given_mean(device):
    q, k, _ = oracle.make_batch(2, 1, 4, 2, 96, 64, Sk=80)
    qo, qso, ko, kso, mo = oracle.quantize_qk(q, k, softmax_scale=0.2)
    q_i8, q_scale, k_i8, k_scale, mean = s8.quantize_qk(q.to(device), k.to(device), softmax_scale=0.2,
                                                        k_mean_override=mo.to(device))
    assert torch.equal(q_i8.cpu(), qo) and torch.equal(q_scale.cpu(), qso)
    assert torch.equal(k_i8.cpu(), ko) and torch.equal(k_scale.cpu(), kso)
    k_s, mean2 = s8.smooth_k(k.to(device))
    assert k_s.shape == k.shape and mean2.shape == (1, 2, 1, 64)


def test_gate_exact_at_the_threshold_boundary(device):
    """Rows whose lower median sits on fp16 neighbours of max/12: the fused statistic (packed
    fp16 path for max/12 >= 2^-7, fp32 path below) must agree with the reference formula row by row."""
    g = torch.Generator().manual_seed(123)
    rows = []
    for amax in [1.0, 3.0, 12.0, 0.75, 100.0, 0.05, 0.011, 6.0e-4, 65504.0, 7.3, 0.0947, 0.0937]:
        a16 = torch.tensor(amax).half()
        c0 = (a16.float() / 12.0).half()
        for step in range(-4, 5):
            c = torch.tensor(c0.view(torch.int16).item() + step, dtype=torch.int16).view(torch.float16)
            row = torch.empty(128, dtype=torch.float16)
            row[:64] = c                       # 64 smallest -> the lower median is c
            row[64:127] = (a16.float() * 0.5).half()
            row[127] = a16
            sign = torch.where(torch.rand(128, generator=g) < 0.5, -1.0, 1.0).half()
            rows.append((row * sign)[torch.randperm(128, generator=g)])
    q = torch.stack(rows)
    expect = oracle.outlier_rows(q)
    assert bool(expect.any()) and not bool(expect.all())
    neg = q[~expect]
    assert s8.detect_q_outlier_domination(neg.view(1, 1, -1, 128).contiguous().to(device)) is False
    for r in q[expect]:
        assert s8.detect_q_outlier_domination(r.view(1, 1, 1, 128).contiguous().to(device)) is True
    # one positive row hidden among many negative ones still trips the any-row flag
    mixed = torch.cat([neg, q[expect][:1], neg])
    assert s8.detect_q_outlier_domination(mixed.view(1, 1, -1, 128).contiguous().to(device)) is True
    # other head dims use other lane layouts
    for D in (64, 256, 80):
        x = torch.randn(3000, D, generator=g).half()
        x[::97, 0] *= 9.0
        e = oracle.outlier_rows(x)
        for lo in range(0, 3000, 500):
            blk = x[lo:lo + 500]
            assert s8.detect_q_outlier_domination(blk.view(1, 1, -1, D).contiguous().to(device)) == bool(e[lo:lo + 500].any())


def test_gate_only_kernel_equals_the_fused_gate(device):
    # the statistic evaluated alone (one read of Q) and inside the quantisation pass must agree
    g = np.load(GOLDEN / "outlier_gate.npz")
    for name in ("clean", "spike", "chan20", "d64", "near"):
        q = from_bits(g[f"{name}__q"], "float16").to(device)
        alone = bool(quant.q_outlier_flag(q).item())
        fused = bool(quant.quantize_q(q, 1.0, want_gate=True)[2].item())
        assert alone == fused == bool(g[f"{name}__flag"]), name
    x = torch.randn(33, 72, device=device)          # fp32 / odd width: generic kernel
    x[5, 3] = 500.0
    assert bool(quant.q_outlier_flag(x).item()) and not bool(quant.q_outlier_flag(torch.randn(33, 72, device=device)).item())


def test_attention_asks_the_gate_first_after_a_demotion(device):
    q, k, v = (t.to(device) for t in oracle.make_batch(91, 1, 4, 2, 128, 64))
    qo = q.clone()
    qo[..., 5] *= 40.0
    a1 = s8.attn_int8_fwd(qo, k, v, causal=True)          # demoted (fused gate)
    assert s8.ops.last_gate_decision is True
    a2 = s8.attn_int8_fwd(qo, k, v, causal=True)          # demoted again (gate asked first)
    assert s8.ops.last_gate_decision is True and torch.equal(a1, a2)
    b1 = s8.attn_int8_fwd(q, k, v, causal=True)           # gate first, passes, then quantise
    assert s8.ops.last_gate_decision is False
    b2 = s8.attn_int8_fwd(q, k, v, causal=True)           # fused gate
    assert torch.equal(b1, b2)


@pytest.mark.parametrize("D,dtype", [(128, torch.float16), (64, torch.float16), (256, torch.bfloat16), (128, torch.bfloat16)])
def test_one_launch_k_prologue_equals_the_two_step_path_bitwise(D, dtype, device):
    # The cluster kernel (mean through distributed shared memory, quantisation on a second walk) keeps the
    # chunked, fixed-order sum of sl8_k_mean: mean, codes, scales and smoothed keys are the same bits.
    g = torch.Generator().manual_seed(500 + D)
    for (B, H, N) in ((1, 2, 1000), (2, 3, 1024), (1, 2, 1025), (1, 1, 5000), (2, 2, 8192), (1, 1, 9217), (1, 2, 7)):
        k = (torch.randn(B, H, N, D, generator=g) + 0.7 * torch.randn(1, H, 1, D, generator=g)).to(dtype).to(device)
        assert _lib.load().sl8_k_prologue_fused_ok(_C._DTYPE[dtype], B * H, N, D) == 1
        mean2 = quant.k_mean(k)
        i2, s2, ks2 = quant.smooth_quantize_k(k, mean2, want_smoothed=True)
        i1, s1, mean1, ks1 = quant.k_prologue(k, want_smoothed=True)
        assert torch.equal(mean1, mean2), (B, H, N)
        assert torch.equal(i1, i2) and torch.equal(s1, s2) and torch.equal(ks1.view(torch.int16), ks2.view(torch.int16)), (B, H, N)
        # repeatable
        j1, t1, m1, _ = quant.k_prologue(k)
        assert torch.equal(j1, i1) and torch.equal(t1, s1) and torch.equal(m1, mean1)
    # per-sequence lengths: the mean runs over the first len keys of each sequence, all rows are quantised
    k = torch.randn(3, 2, 3000, D, generator=g).to(dtype).to(device)
    lens = torch.tensor([3000, 17, 1500], dtype=torch.int32, device=device)
    mean2 = quant.k_mean(k, lens)
    i2, s2, _ = quant.smooth_quantize_k(k, mean2)
    i1, s1, mean1, _ = quant.k_prologue(k, lens)
    assert torch.equal(mean1, mean2) and torch.equal(i1, i2) and torch.equal(s1, s2)
    # shapes the cluster kernel does not serve fall back to the two steps
    k = torch.randn(1, 2, 300, 80, generator=g).to(dtype).to(device)
    assert _lib.load().sl8_k_prologue_fused_ok(_C._DTYPE[dtype], 2, 300, 80) == 0
    i1, s1, mean1, _ = quant.k_prologue(k)
    assert torch.equal(mean1, quant.k_mean(k)) and torch.equal(i1, quant.smooth_quantize_k(k, mean1)[0])


# ---- rotate=True prologue: Hadamard rotation in the row quantiser's registers ----------------

def _ulp_close(a: torch.Tensor, b: torch.Tensor, x: torch.Tensor, frac_exact: float) -> None:
    """a and b are roundings of the same rotation of x computed in two summation orders: equal but for
    a few elements that sat on a rounding boundary; those differ by one unit in the last place plus the
    fp32 error of a sum of the row's terms (which counts where the terms cancel to something small)."""
    a, b = a.cpu(), b.cpu()
    assert a.dtype == b.dtype and a.shape == b.shape
    same = (a == b).float().mean().item()
    assert same >= frac_exact, same
    step = torch.maximum(a.float().abs(), b.float().abs()) * (2.0 ** -10 if a.dtype == torch.float16 else 2.0 ** -7)
    sum_err = x.float().abs().sum(-1, keepdim=True) / x.shape[-1] ** 0.5 * 2.0 ** -20
    assert bool(((a.float() - b.float()).abs() <= step + sum_err + 1e-7).all())


@pytest.mark.parametrize("D", [32, 64, 128, 256, 512])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_hadamard_rotation_kernel_against_the_matmul_formula(D, dtype, device):
    x = (torch.randn(3, 5, 77, D, generator=torch.Generator().manual_seed(D)) * 2.0).to(dtype)
    x[0, 0, 3] = 0
    x[1, 2, 5, 7] = 300.0
    got = quant.rotate_last(x.to(device))
    assert got.dtype == dtype and got.shape == x.shape
    _ulp_close(got, oracle.rotate_last(x), x, 0.97)
    # orthonormal: rotating twice gives the input back (to the rounding of the two casts)
    back = quant.rotate_last(got)
    tol = 2e-3 if dtype == torch.float16 else 2e-2
    assert torch.allclose(back.float().cpu(), x.float(), atol=tol * float(x.float().abs().max()), rtol=tol)
    assert torch.equal(got, quant.rotate_last(x.to(device)))           # bitwise repeatable


def test_hadamard_rotation_golden_vectors(device):
    g = np.load(GOLDEN / "rotation.npz")
    for name, dt in (("f16_128", "float16"), ("bf16_64", "bfloat16"), ("f16_32", "float16")):
        x = from_bits(g[f"{name}__x"], dt)
        _ulp_close(quant.rotate_last(x.to(device)), from_bits(g[f"{name}__rot"], dt), x, 0.97)


@pytest.mark.parametrize("D", [64, 128, 256])
def test_rotated_quantize_qk_is_the_oracles_up_to_the_rotation_order(D, device):
    gen = torch.Generator().manual_seed(700 + D)
    q = torch.randn(2, 4, 150, D, generator=gen).half()
    k = torch.randn(2, 2, 190, D, generator=gen).half() + 0.5
    k[..., 5] *= 12.0
    oq_i8, oq_s, ok_i8, ok_s, omean = oracle.quantize_qk(q, k, rotate=True)
    q_i8, q_s, k_i8, k_s, mean = quant.quantize_qk(q.to(device), k.to(device), rotate=True, k_mean_override=omean.to(device))
    assert q_i8.shape == oq_i8.shape and q_s.shape == oq_s.shape and k_i8.shape == ok_i8.shape and k_s.shape == ok_s.shape
    # a rotated value that rounds the other way moves its code by at most one and the row scale by one fp16 step
    for got, ref in ((q_i8, oq_i8), (k_i8, ok_i8)):
        d = (got.cpu().int() - ref.int()).abs()
        assert int(d.max()) <= 1 and float((d != 0).float().mean()) < 0.02
    for got, ref in ((q_s, oq_s), (k_s, ok_s)):
        assert torch.allclose(got.cpu(), ref, rtol=1.1e-3, atol=0)
    # the kernel's own pieces agree with each other bit for bit: rotation alone, then the plain quantiser
    k_sm = quant.smooth_quantize_k(k.to(device), omean.to(device), want_smoothed=True)[2]
    r_i8, r_s = quant.quantize_int8_rowwise(quant.rotate_last(k_sm))
    assert torch.equal(r_i8, k_i8) and torch.equal(r_s, k_s)
    # and attention through the rotated prologue keeps the int8 quality bar
    v = torch.randn(2, 2, 190, D, generator=gen).half()
    out = s8.attn_int8_fwd(q.to(device), k.to(device), v.to(device), rotate=True, internal_accuracy_gate=False)
    oracle.assert_int8_quality(out, oracle.attention_fp32(q, k, v), what=f"rotated prologue D={D}")


def test_hadamard_entry_rejects_what_it_cannot_rotate(device):
    x = torch.randn(4, 96, device=device).half()
    with pytest.raises(RuntimeError, match="power-of-two"):
        quant.hadamard_quantize_rows(x)
    with pytest.raises(ValueError, match="power-of-two"):
        quant.rotate_last(x)
    f = torch.randn(4, 64, device=device)                  # fp32: the matmul formula in torch
    assert torch.allclose(quant.rotate_last(f).cpu(), oracle.rotate_last(f.cpu()), atol=1e-5)
