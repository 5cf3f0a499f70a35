"""Backward kernels (dQ pass, dK/dV pass; tcgen05 for D = 64 / 128 and the mma.sync pair for
every D) against the CPU restatement of the reference's exact gradient, through the C ABI.  Bars: the reference's own for its CUDA backward are cos >= 0.99,
rel-L1 <= 0.06, SQNR >= 14 dB (tests/test_attn_bwd_cuda.py:24); this path contracts in 16-bit
with fp32 accumulation and is held to cos >= 0.9999, rel-L1 <= 0.01, SQNR >= 40 dB."""

import numpy as np
import pytest
import torch

import superl8_b200 as s8
from conftest import GOLDEN, from_bits
from oracle import oracle
from superl8_b200 import _C, _lib

pytestmark = pytest.mark.gpu

TC, MMA = _lib.SL8_BACKEND_TCGEN05, _lib.SL8_BACKEND_MMA


def _backends(D):
    return (TC, MMA) if D in (64, 128) else (MMA,)

BARS = dict(min_cos=0.9999, max_rel_l1=0.01, min_sqnr_db=40.0)


def _check(got, ref, what):
    assert got.shape == ref.shape, what
    c, l1, s = oracle.cos_sim(got, ref), oracle.rel_l1(got, ref), oracle.sqnr_db(got, ref)
    assert c >= BARS["min_cos"] and l1 <= BARS["max_rel_l1"] and s >= BARS["min_sqnr_db"], (what, c, l1, s)


def test_golden_gradients(device):
    g = np.load(GOLDEN / "attn_backward.npz")
    for name in ("mha", "mha_causal", "rect_causal", "gqa_causal", "mqa"):
        q, k, v, o, do = (from_bits(g[f"{name}__{n}"], "float16").to(device) for n in ("q", "k", "v", "o", "do"))
        causal, scale = bool(g[f"{name}__cfg"][0]), float(g[f"{name}__cfg"][1])
        lse = torch.from_numpy(g[f"{name}__lse"]).to(device)
        for backend in _backends(q.shape[-1]):
            dq, dk, dv = _C.attn_bwd(q, k, v, o, do, lse, scale, causal, backend=backend)
            assert dq.dtype == torch.float16 and dk.shape == k.shape and dv.shape == v.shape
            for got, key in ((dq, "dq"), (dk, "dk"), (dv, "dv")):
                _check(got, torch.from_numpy(g[f"{name}__{key}"]), (name, key, backend))
        assert _C.device_status() == 0


# the reference's shapes (tests/test_attn_bwd_cuda.py:23) plus grouped heads, ragged sizes, D = 32,
# and sequences of several 128-wide tiles (the stage ring of the tensor-memory passes wraps)
SHAPES = [(1, 2, 2, 128, 128, 64), (2, 4, 4, 256, 256, 64), (1, 2, 2, 257, 257, 64), (1, 2, 2, 192, 192, 128),
          (1, 8, 2, 200, 200, 128), (2, 4, 1, 100, 333, 32), (1, 2, 1, 300, 70, 64), (1, 4, 2, 650, 650, 128),
          (1, 2, 1, 520, 900, 64), (1, 2, 2, 900, 520, 128)]


@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("causal", [False, True])
def test_backward_matches_oracle(device, shape, causal):
    B, Hq, Hkv, M, N, D = shape
    gen = torch.Generator().manual_seed(1000 + M + N + D)
    q = torch.randn(B, Hq, M, D, generator=gen).half()
    k = torch.randn(B, Hkv, N, D, generator=gen).half()
    v = torch.randn(B, Hkv, N, D, generator=gen).half()
    do = torch.randn(B, Hq, M, D, generator=gen).half()
    out, lse = _C.attn_fp16_fwd(q.to(device), k.to(device), v.to(device), causal, None, want_lse=True)
    rq, rk, rv = oracle.attention_backward_fp32(q, k, v, out, do, causal)
    for backend in _backends(D):
        dq, dk, dv = s8.backward_cuda(q.to(device), k.to(device), v.to(device), out, lse, do.to(device), causal=causal,
                                      backend=backend)
        assert _C.device_status() == 0
        for got, ref, key in ((dq, rq, "dq"), (dk, rk, "dk"), (dv, rv, "dv")):
            assert torch.isfinite(got.float()).all(), (shape, causal, key, backend)
            _check(got, ref, (shape, causal, key, backend))
    # lse omitted: produced by the forward kernel; same result (same backend: the default one)
    dq1, dk1, dv1 = s8.backward_cuda(q.to(device), k.to(device), v.to(device), out, lse, do.to(device), causal=causal)
    dq2, dk2, dv2 = s8.backward_cuda(q.to(device), k.to(device), v.to(device), out, None, do.to(device), causal=causal)
    assert torch.equal(dq1, dq2) and torch.equal(dk1, dk2) and torch.equal(dv1, dv2)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_backward_with_large_logits(device, dtype):
    """Peaked attention rows (logits of a few tens, lse far from 0) and a row-sum gradient
    with a large mean: the tensor-memory passes carry -lse / scale and -D_m of a query as a
    {hi, lo} 16-bit pair on an extra step of the S and dP contractions, which has to stay exact
    enough for both dtypes."""
    gen = torch.Generator().manual_seed(4242)
    B, Hq, Hkv, M, N, D = 1, 4, 2, 384, 384, 128
    q = (3.0 * torch.randn(B, Hq, M, D, generator=gen)).to(dtype)
    k = (3.0 * torch.randn(B, Hkv, N, D, generator=gen)).to(dtype)
    v = (torch.randn(B, Hkv, N, D, generator=gen) + 2.0).to(dtype)
    do = (torch.randn(B, Hq, M, D, generator=gen) + 1.0).to(dtype)
    for causal in (False, True):
        out, lse = _C.attn_fp16_fwd(q.to(device), k.to(device), v.to(device), causal, None, want_lse=True)
        assert float(lse.abs().max()) > 20.0
        ref = oracle.attention_backward_fp32(q, k, v, out, do, causal)
        got_tc = s8.backward_cuda(q.to(device), k.to(device), v.to(device), out, lse, do.to(device), causal=causal, backend=TC)
        got_mma = s8.backward_cuda(q.to(device), k.to(device), v.to(device), out, lse, do.to(device), causal=causal, backend=MMA)
        assert _C.device_status() == 0
        for a, b, r, key in zip(got_tc, got_mma, ref, ("dq", "dk", "dv")):
            assert torch.isfinite(a.float()).all()
            if dtype == torch.float16:
                _check(a, r, ("large logits", causal, key))
            else:
                assert oracle.cos_sim(a, r) >= 0.999 and oracle.rel_l1(a, r) <= 0.03, (causal, key)
            # and no further from the oracle than the warp-level kernels are
            assert oracle.rel_l1(a, r) <= 1.5 * oracle.rel_l1(b, r) + 1e-4, (causal, key, oracle.rel_l1(a, r), oracle.rel_l1(b, r))


def test_backward_is_deterministic_and_bf16(device):
    # reference tests/test_attn_bwd_cuda.py:88-96: atomic-free -> bitwise reproducible
    gen = torch.Generator().manual_seed(77)
    q, k, v, do = (torch.randn(2, 4, 256, 64, generator=gen).half().to(device) for _ in range(4))
    out, lse = _C.attn_fp16_fwd(q, k, v, False, None, want_lse=True)
    qb, kb, vb, dob = (t.bfloat16() for t in (q, k, v, do))
    outb, lseb = _C.attn_fp16_fwd(qb, kb, vb, True, None, want_lse=True)
    ref = oracle.attention_backward_fp32(qb, kb, vb, outb, dob, True)
    for backend in (TC, MMA):
        r0 = s8.backward_cuda(q, k, v, out, lse, do, backend=backend)
        for _ in range(3):
            for a, b in zip(s8.backward_cuda(q, k, v, out, lse, do, backend=backend), r0):
                assert torch.equal(a, b)
        got = s8.backward_cuda(qb, kb, vb, outb, lseb, dob, causal=True, backend=backend)
        for a, b in zip(got, ref):
            assert a.dtype == torch.bfloat16 and oracle.cos_sim(a, b) >= 0.999 and oracle.rel_l1(a, b) <= 0.03
    assert _C.device_status() == 0


def test_backward_edge_cases_and_errors(device):
    z = torch.zeros(1, 2, 0, 64, dtype=torch.float16, device=device)
    kv = torch.randn(1, 2, 40, 64, device=device).half()
    dq, dk, dv = _C.attn_bwd(z, kv, kv, z, z, torch.zeros(1, 2, 0, device=device), 0.125, False)
    assert dq.numel() == 0 and float(dk.abs().max()) == 0.0 and float(dv.abs().max()) == 0.0
    q = torch.randn(1, 2, 8, 64, device=device).half()
    e = torch.zeros(1, 2, 0, 64, dtype=torch.float16, device=device)
    dq, dk, dv = _C.attn_bwd(q, e, e, q, q, torch.zeros(1, 2, 8, device=device), 0.125, False)
    assert float(dq.abs().max()) == 0.0 and dk.numel() == 0
    with pytest.raises(RuntimeError, match="head dim"):
        x = torch.zeros(1, 1, 16, 96, dtype=torch.float16, device=device)
        _C.attn_bwd(x, x, x, x, x, torch.zeros(1, 1, 16, device=device), 0.1, False)
    with pytest.raises(RuntimeError, match="float16"):
        x = torch.zeros(1, 1, 16, 64, dtype=torch.float32, device=device)
        _C.attn_bwd(x, x, x, x, x, torch.zeros(1, 1, 16, device=device), 0.1, False)
    with pytest.raises(RuntimeError, match="float32"):
        x = torch.zeros(1, 1, 16, 64, dtype=torch.float16, device=device)
        _C.attn_bwd(x, x, x, x, x, torch.zeros(1, 1, 16, dtype=torch.float16, device=device), 0.1, False)


def test_autograd_uses_the_kernels(device):
    q, k, v = (t.to(device).requires_grad_(True) for t in oracle.make_batch(46, 1, 4, 2, 160, 64))
    before = s8._lib.launches
    out = s8.attn(q, k, v, causal=True)
    out.backward(torch.ones_like(out))
    assert s8._lib.launches - before >= 3
    rq, rk, rv = oracle.attention_backward_fp32(q, k, v, out.detach(), torch.ones_like(out), True)
    for a, b in ((q.grad, rq), (k.grad, rk), (v.grad, rv)):
        assert oracle.cos_sim(a, b) >= 0.99     # the forward is the int8 one: the reference's bar


def test_autograd_with_a_per_channel_key_offset(device):
    # K smoothing exists for keys with a per-channel mean.  The int8 forward sees k - mean, so its
    # row statistic lacks scale * q.mean; the wrapper adds it back before the backward (which
    # recomputes the logits from the unsmoothed k).  Without that every row of P is off by
    # exp(scale * q.mean) and all three gradients are wrong.
    q, k, v = oracle.make_batch(47, 1, 4, 2, 192, 64)
    g = torch.Generator().manual_seed(470)
    k = (k.float() + 3.0 * torch.randn(1, 2, 1, 64, generator=g)).half()
    qd, kd, vd = (t.to(device).requires_grad_(True) for t in (q, k, v))
    out = s8.attn(qd, kd, vd, causal=True)
    d_out = torch.randn(out.shape, generator=g).half()
    out.backward(d_out.to(device))
    oracle.assert_int8_quality(out.detach(), oracle.attention_fp32(q, k, v, causal=True), what="offset-K forward")
    rq, rk, rv = oracle.attention_backward_fp32(q, k, v, out.detach(), d_out, True)
    for name, a, b in (("dq", qd.grad, rq), ("dk", kd.grad, rk), ("dv", vd.grad, rv)):
        assert oracle.cos_sim(a, b) >= 0.99 and oracle.rel_l1(a, b) <= 0.06, (name, oracle.cos_sim(a, b), oracle.rel_l1(a, b))


def test_attn_ref_shares_the_analytic_backward(device):
    # reference superl8/autograd.py:77-108: plain forward + the same gradient formulas, gradcheck-able
    q, k, v = (torch.randn(1, 2, 6, 8, dtype=torch.float64, device=device, requires_grad=True) for _ in range(3))
    assert torch.autograd.gradcheck(lambda a, b, c: s8.attn_ref(a, b, c, causal=True), (q, k, v))
    assert torch.autograd.gradcheck(lambda a, b, c: s8.attn_ref(a, b, c, scale=0.3), (q, k, v))
