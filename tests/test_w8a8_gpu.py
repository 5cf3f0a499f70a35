"""Full-W8A8 forward (int8 Q.K^T and int8 P.V) through the C ABI: against the reference's own
kernel on the same int8 inputs, against the tile-by-tile oracle, and against fp32 attention with
the reference's bars for this route (tests/test_attn_fwd_w8a8.py:37: cos >= 0.998, rel-L1 <= 0.03,
SQNR >= 18 dB)."""

import pytest
import torch

import superl8_b200 as s8
from gpu_helpers import ref_attn_w8a8_fwd, ref_lib
from oracle import oracle
from superl8_b200 import _C, _lib

pytestmark = pytest.mark.gpu
PV_BARS = dict(min_cos=0.998, max_rel_l1=0.03, min_sqnr_db=18.0)

CASES = [  # B, Hq, Hkv, M, N, D, causal
    (1, 2, 2, 128, 128, 64, False), (2, 4, 2, 257, 257, 64, True), (1, 8, 2, 200, 200, 128, True),
    (1, 4, 1, 70, 333, 32, False), (1, 2, 2, 40, 300, 128, True), (1, 2, 1, 130, 130, 256, True),
]


BACKENDS = {"tensor-memory": _lib.SL8_BACKEND_TCGEN05, "mma.sync": _lib.SL8_BACKEND_MMA}


@pytest.mark.parametrize("case", CASES)
@pytest.mark.parametrize("per_warp", [True, False])
@pytest.mark.parametrize("backend", list(BACKENDS))
def test_w8a8_matches_reference_kernel_and_oracle(device, case, per_warp, backend):
    B, Hq, Hkv, M, N, D, causal = case
    if backend == "tensor-memory" and D == 32:
        pytest.skip("the tensor-memory kernel serves D = 64, 128, 256")
    backend = BACKENDS[backend]
    q, k, v = oracle.make_batch(300 + D, B, Hq, Hkv, M, D, Sk=N)
    q_i8, q_scale, k_i8, k_scale, _ = oracle.quantize_qk(q, k)
    v_i8, v_scale = oracle.quantize_v_perchannel(v)
    qs, ks, vs = q_scale.squeeze(-1).contiguous(), k_scale.squeeze(-1).contiguous(), v_scale.squeeze(-2).contiguous()
    diag = (N - M) if causal else 0
    dv = lambda t: t.to(device)
    out = _C.attn_w8a8_fwd(dv(q_i8), dv(qs), dv(k_i8), dv(ks), dv(v_i8), dv(vs), causal, diag, per_warp, backend=backend)
    assert out.shape == (B, Hq, M, D) and out.dtype == torch.float16
    assert torch.equal(out, _C.attn_w8a8_fwd(dv(q_i8), dv(qs), dv(k_i8), dv(ks), dv(v_i8), dv(vs), causal, diag, per_warp, backend=backend))
    ref_o = oracle.attn_w8a8_fwd(q_i8, qs, k_i8, ks, v_i8, vs, causal, diag, per_warp)
    # same tiles, same scales: only the rounding of an occasional P code (ex2 approximation) differs --
    # and, on the tensor-memory kernel, the fp16 rounding of code * p_scale (2^-11 relative)
    assert oracle.cos_sim(out, ref_o) >= 0.9999 and oracle.rel_l1(out, ref_o) <= 5e-3
    if ref_lib() is not None and D <= 128:
        ref_k = ref_attn_w8a8_fwd(dv(q_i8), dv(qs), dv(k_i8), dv(ks), dv(v_i8), dv(vs), causal, diag, per_warp)
        assert oracle.cos_sim(out, ref_k) >= 0.9999 and oracle.rel_l1(out, ref_k) <= 5e-3
    oracle.assert_int8_quality(out, oracle.attention_fp32(q, k, v, causal=causal), what=f"w8a8 {case}", **PV_BARS)


def test_public_int8_pv_route(device):
    q, k, v = (t.to(device) for t in oracle.make_batch(310, 2, 4, 2, 300, 128))
    out = s8.attn_int8_fwd(q, k, v, causal=True, int8_pv=True)
    ref = oracle.attention_fp32(q, k, v, causal=True)
    oracle.assert_int8_quality(out, ref, what="public w8a8", **PV_BARS)
    fp16pv = s8.attn_int8_fwd(q, k, v, causal=True, internal_accuracy_gate=False)
    assert oracle.rel_l1(fp16pv, ref) <= oracle.rel_l1(out, ref) + 1e-4   # the reference's ladder
    with pytest.raises(ValueError, match="window_left"):
        s8.attn_int8_fwd(q, k, v, int8_pv=True, window_left=16)
    with pytest.raises(RuntimeError, match="head dim"):
        z = torch.zeros(1, 1, 8, 96, dtype=torch.int8, device=device)
        _C.attn_w8a8_fwd(z, torch.zeros(1, 1, 8, device=device), z, torch.zeros(1, 1, 8, device=device), z,
                         torch.zeros(1, 1, 96, device=device))


def test_int8_pv_is_still_behind_the_accuracy_gate(device):
    # The reference asks its gate before it looks at int8_pv (superl8/ops.py:121 precedes :152): an
    # outlier-dominated Q demotes the call to the full-precision kernel on the int8_pv route too.
    q, k, v = oracle.make_batch(311, 1, 4, 2, 200, 128)
    q[0, 1, 17, 5] = 70.0
    assert oracle.detect_q_outlier_domination(q)
    ref = oracle.attention_fp32(q, k, v, causal=True)
    out = s8.attn_int8_fwd(q.to(device), k.to(device), v.to(device), causal=True, int8_pv=True)
    assert s8.ops.last_gate()[0] is True
    assert oracle.cos_sim(out, ref) >= 0.9999 and oracle.rel_l1(out, ref) <= 5e-3      # the full-precision bar
    # demoted calls keep the window (the reference returns before its int8_pv window check)
    outw = s8.attn_int8_fwd(q.to(device), k.to(device), v.to(device), causal=True, int8_pv=True, window_left=64)
    refw = oracle.attention_fp32(q, k, v, causal=True, window_left=64)
    assert oracle.cos_sim(outw, refw) >= 0.9999
    # gate off: the W8A8 kernel runs whatever Q looks like
    out2 = s8.attn_int8_fwd(q.to(device), k.to(device), v.to(device), causal=True, int8_pv=True,
                            internal_accuracy_gate=False)
    assert s8.ops.last_gate()[0] is None and torch.isfinite(out2.float()).all()
    assert not torch.equal(out2, out)


def test_w8a8_backends_agree_and_the_causal_diagonal_picks_the_kernel(device):
    """Both kernels form the same int8 grid for P; a causal diagonal that is not at the sequence
    end (only the mma.sync kernel takes one) is routed there and refused by the other."""
    q, k, v = oracle.make_batch(320, 2, 4, 2, 300, 128)
    q_i8, q_scale, k_i8, k_scale, _ = oracle.quantize_qk(q, k)
    v_i8, v_scale = oracle.quantize_v_perchannel(v)
    args = [t.to(device) for t in (q_i8, q_scale.squeeze(-1).contiguous(), k_i8, k_scale.squeeze(-1).contiguous(), v_i8,
                                   v_scale.squeeze(-2).contiguous())]
    tc = _C.attn_w8a8_fwd(*args, True, 0, True, backend=_lib.SL8_BACKEND_TCGEN05)
    mma = _C.attn_w8a8_fwd(*args, True, 0, True, backend=_lib.SL8_BACKEND_MMA)
    assert oracle.cos_sim(tc, mma) >= 0.99999 and oracle.rel_l1(tc, mma) <= 2e-3
    assert torch.equal(_C.attn_w8a8_fwd(*args, True, 0, True), tc)            # the default where it serves
    shifted = _C.attn_w8a8_fwd(*args, True, 5, True)
    assert torch.equal(shifted, _C.attn_w8a8_fwd(*args, True, 5, True, backend=_lib.SL8_BACKEND_MMA))
    with pytest.raises(RuntimeError, match="does not serve"):
        _C.attn_w8a8_fwd(*args, True, 5, True, backend=_lib.SL8_BACKEND_TCGEN05)
    assert _C.device_status(device) == 0
