"""Pins oracle/oracle.py against vectors produced by the reference's own Python code
(tests/golden/make_golden.py).  CPU only."""

import numpy as np
import torch

from conftest import GOLDEN, from_bits
from oracle import oracle


def test_quantize_rowwise_matches_reference_cpu_branch():
    g = np.load(GOLDEN / "quant_rowwise.npz")
    names = sorted({k.split("__")[0] for k in g.files})
    assert len(names) == 6
    for n in names:
        x = from_bits(g[f"{n}__x"], str(g[f"{n}__dtype"]))
        q, s = oracle.quantize_rowwise(x, rule="cpu")
        assert np.array_equal(q.numpy(), g[f"{n}__q"]), n
        assert np.array_equal(s.numpy(), g[f"{n}__scale"]), n


def test_cuda_rule_differs_from_cpu_rule_only_through_the_scale():
    # scale = amax * f32(1/127) vs amax / 127: at most 1 ulp apart; where the two scales
    # agree the codes agree (same division, same rounding).
    g = np.load(GOLDEN / "quant_rowwise.npz")
    x = from_bits(g["f16_128__x"], "float16")
    qc, sc = oracle.quantize_rowwise(x, rule="cuda")
    qr, sr = g["f16_128__q"], g["f16_128__scale"]
    same = (sc.numpy() == sr).reshape(-1)
    assert same.sum() >= 1
    assert np.array_equal(qc.numpy()[same], qr[same])
    rel = np.abs(sc.numpy() - sr) / sr
    assert rel.max() <= 2.0 ** -22
    assert np.abs(qc.numpy().astype(int) - qr.astype(int)).max() <= 1
    assert qc.numpy().min() >= -127 and sc.numpy()[3, 0] == 1.0 and np.all(qc.numpy()[3] == 0)


def test_smooth_k_bit_exact():
    g = np.load(GOLDEN / "smooth_k.npz")
    for n in ("short", "chunked", "bf16"):
        dt = str(g[f"{n}__dtype"])
        k = from_bits(g[f"{n}__k"], dt)
        k_s, mean = oracle.smooth_k(k)
        assert np.array_equal(mean.numpy(), g[f"{n}__k_mean"]), n
        assert torch.equal(k_s, from_bits(g[f"{n}__k_s"], dt)), n


def test_outlier_gate():
    g = np.load(GOLDEN / "outlier_gate.npz")
    expect = {"clean": False, "spike": True, "chan20": True, "near": True}
    for n in ("clean", "spike", "chan20", "d64", "near"):
        q = from_bits(g[f"{n}__q"], "float16")
        assert oracle.detect_q_outlier_domination(q) == bool(g[f"{n}__flag"]), n
        if n in expect:
            assert bool(g[f"{n}__flag"]) == expect[n]
        rows = oracle.outlier_rows(q).numpy()
        assert np.array_equal(rows, g[f"{n}__ratio"] > 12.0)
    near = oracle.outlier_rows(from_bits(g["near__q"], "float16")).numpy().reshape(-1)
    assert list(near) == [False, True, False, False]   # ratio exactly 12 does not trip the gate


def test_quantize_qk_matches_reference_cpu_branch():
    g = np.load(GOLDEN / "quantize_qk.npz")
    q, k = from_bits(g["q"], "float16"), from_bits(g["k"], "float16")
    for name, sc in (("default", None), ("scaled", 0.2)):
        q_i8, q_scale, k_i8, k_scale, k_mean = oracle.quantize_qk(q, k, softmax_scale=sc, rule="cpu")
        assert np.array_equal(q_i8.numpy(), g[f"{name}__q_i8"])
        assert np.array_equal(q_scale.numpy(), g[f"{name}__q_scale"])
        assert np.array_equal(k_i8.numpy(), g[f"{name}__k_i8"])
        assert np.array_equal(k_scale.numpy(), g[f"{name}__k_scale"])
        assert np.array_equal(k_mean.numpy(), g[f"{name}__k_mean"])


def test_hadamard_rotation_and_rotated_quantize_qk_match_the_reference():
    g = np.load(GOLDEN / "rotation.npz")
    for name, dt in (("f16_128", "float16"), ("bf16_64", "bfloat16"), ("f16_32", "float16")):
        x = from_bits(g[f"{name}__x"], dt)
        assert torch.equal(oracle.rotate_last(x), from_bits(g[f"{name}__rot"], dt))
    q, k = from_bits(g["q"], "float16"), from_bits(g["k"], "float16")
    q_i8, q_scale, k_i8, k_scale, k_mean = oracle.quantize_qk(q, k, rule="cpu", rotate=True)
    for got, key in ((q_i8, "q_i8"), (q_scale, "q_scale"), (k_i8, "k_i8"), (k_scale, "k_scale"), (k_mean, "k_mean")):
        assert np.array_equal(got.numpy(), g[key]), key


def test_fp32_attention_oracles():
    g = np.load(GOLDEN / "attention_fp32.npz")
    q, k, v = (from_bits(g[n], "float16") for n in ("q", "k", "v"))
    assert np.array_equal(oracle.attention_fp32(q, k, v).numpy(), g["noncausal"])
    assert np.array_equal(oracle.attention_fp32(q, k, v, causal=True).numpy(), g["causal_rect"])
    assert np.array_equal(oracle.attention_fp32(q, k, v, causal=True, scale=0.3).numpy(), g["scaled"])
    assert np.array_equal(oracle.attention_fp32(q, k, v, window_left=9).numpy(), g["window9"])
    a, b = torch.from_numpy(g["metric_a"]), torch.from_numpy(g["metric_b"])
    vals = np.array([oracle.cos_sim(b, a), oracle.rel_l1(b, a), oracle.sqnr_db(b, a)])
    assert np.array_equal(vals, g["metric_vals"])


def test_kernel_restatement_meets_the_reference_gate_on_clean_data():
    # int8 kernel mathematics (restated) vs the fp32 oracle, reference tolerance gate.
    q, k, v = oracle.make_batch(1, 1, 4, 2, 160, 64)
    q_i8, q_scale, k_i8, k_scale, _ = oracle.quantize_qk(q, k)
    for causal in (False, True):
        out = oracle.attn_int8_fwd(q_i8, q_scale.squeeze(-1), k_i8, k_scale.squeeze(-1), v, causal=causal)
        oracle.assert_int8_quality(out, oracle.attention_fp32(q, k, v, causal=causal))


def test_decode_restatement_split_invariance_and_prefill_agreement():
    q, k, v = oracle.make_batch(5, 2, 8, 2, 1, 64, Sk=333)
    q_i8, q_scale, k_i8, k_scale, _ = oracle.quantize_qk(q, k)
    ref = oracle.attention_fp32(q, k, v)
    outs = [oracle.attn_int8_decode(q_i8, q_scale, k_i8, k_scale.squeeze(-1), v, n_splits=ns) for ns in (1, 3, 16)]
    for o in outs:
        oracle.assert_int8_quality(o, ref)
        assert oracle.cos_sim(o, outs[0]) >= 0.99999
    pre = oracle.attn_int8_fwd(q_i8, q_scale.squeeze(-1), k_i8, k_scale.squeeze(-1), v)
    assert oracle.cos_sim(outs[0], pre) >= 0.999
    lens = torch.tensor([100, 333])
    rag = oracle.attn_int8_decode(q_i8, q_scale, k_i8, k_scale.squeeze(-1), v, n_splits=4, context_lens=lens)
    short = oracle.attn_int8_decode(q_i8[:1], q_scale[:1], k_i8[:1, :, :100], k_scale.squeeze(-1)[:1, :, :100],
                                    v[:1, :, :100], n_splits=1)
    assert oracle.cos_sim(rag[:1], short) >= 0.99999


def test_choose_n_splits_reference_values():
    assert oracle.choose_n_splits_reference(0, 8) == 1
    assert oracle.choose_n_splits_reference(32768, 8192) == 128
    assert oracle.choose_n_splits_reference(64000, 24) == 250
    assert oracle.choose_n_splits_reference(100000, 24) == 256
    assert oracle.choose_n_splits_reference(100, 8) == 3


def test_backward_restatement_matches_the_reference_gradients():
    # reference superl8/autograd.py::_attn_backward (equal head counts) and autograd through its
    # fp32 oracle (grouped heads); P from the saved row sums and P from softmax must agree too.
    g = np.load(GOLDEN / "attn_backward.npz")
    for name in ("mha", "mha_causal", "rect_causal", "gqa_causal", "mqa"):
        q, k, v, o, do = (from_bits(g[f"{name}__{n}"], "float16") for n in ("q", "k", "v", "o", "do"))
        causal, scale = bool(g[f"{name}__cfg"][0]), float(g[f"{name}__cfg"][1])
        lse = torch.from_numpy(g[f"{name}__lse"])
        assert torch.allclose(oracle.attention_lse_fp32(q, k, causal, scale), lse, rtol=0, atol=2e-6), name
        for use_lse in (None, lse):
            dq, dk, dv = oracle.attention_backward_fp32(q, k, v, o, do, causal, scale, lse=use_lse)
            for got, key in ((dq, "dq"), (dk, "dk"), (dv, "dv")):
                ref = torch.from_numpy(g[f"{name}__{key}"])
                assert got.shape == ref.shape
                # grouped-head goldens come from autograd through the fp32 oracle, which never
                # rounds O to fp16; the analytic form reads the stored fp16 O in D = sum(dO * O)
                tol = 2e-5 if name.startswith(("mha", "rect")) else 2e-3
                assert float((got - ref).abs().max()) <= tol * max(1.0, float(ref.abs().max())), (name, key)


def test_varlen_k_prologue_matches_the_reference():
    # reference superl8/ops.py::_varlen_smooth_k (ragged and equal-length branches) + its row quantiser
    g = np.load(GOLDEN / "varlen_prologue.npz")
    for name in ("ragged", "equal"):
        k = from_bits(g[f"{name}__k"], "float16")
        cu = g[f"{name}__cu"]
        k_s = oracle.varlen_smooth_k(k, cu)
        assert np.array_equal(k_s.view(torch.int16).numpy(), g[f"{name}__k_s"]), name
        q, s = oracle.quantize_rowwise(k_s, rule="cpu")
        assert np.array_equal(q.numpy(), g[f"{name}__k_i8"]) and np.array_equal(s.numpy(), g[f"{name}__k_scale"]), name


def test_varlen_restatement_equals_the_dense_one_per_sequence():
    # one packed sequence == the dense restatement on that sequence
    q, k, v = oracle.make_batch(7, 1, 4, 2, 90, 64, Sk=130)
    pk = lambda t: t[0].transpose(0, 1).contiguous()
    cu_q, cu_k = [0, 90], [0, 130]
    out = oracle.attn_int8_varlen(pk(q), pk(k), pk(v), cu_q, cu_k, causal=True)
    q_i8, q_scale, k_i8, k_scale, _ = oracle.quantize_qk(q, k)
    ref = oracle.attn_int8_fwd(q_i8, q_scale.squeeze(-1), k_i8, k_scale.squeeze(-1), v, causal=True)
    assert oracle.cos_sim(out, pk(ref)) >= 0.99999


def test_v_perchannel_quantiser_matches_the_reference():
    g = np.load(GOLDEN / "v_perchannel.npz")
    for name in ("f16", "bf16"):
        v = from_bits(g[f"{name}__v"], str(g[f"{name}__dtype"]))
        v_i8, v_scale = oracle.quantize_v_perchannel(v)
        assert np.array_equal(v_i8.numpy(), g[f"{name}__v_i8"]) and np.array_equal(v_scale.numpy(), g[f"{name}__v_scale"])


def test_w8a8_restatement_quality_and_ladder():
    # reference tests/test_attn_fwd_w8a8.py:37-75: the int8-P.V route meets its own bars against
    # the fp32 oracle and is no better than the fp16-P.V route
    q, k, v = oracle.make_batch(9, 1, 4, 2, 150, 64)
    q_i8, q_scale, k_i8, k_scale, _ = oracle.quantize_qk(q, k)
    v_i8, v_scale = oracle.quantize_v_perchannel(v)
    ref = oracle.attention_fp32(q, k, v, causal=True)
    for per_warp in (True, False):
        out = oracle.attn_w8a8_fwd(q_i8, q_scale.squeeze(-1), k_i8, k_scale.squeeze(-1), v_i8, v_scale.squeeze(-2),
                                   causal=True, causal_diag=0, per_warp=per_warp)
        oracle.assert_int8_quality(out, ref, min_cos=0.998, max_rel_l1=0.03, min_sqnr_db=18.0, what=f"w8a8 {per_warp}")
    fp16pv = oracle.attn_int8_fwd(q_i8, q_scale.squeeze(-1), k_i8, k_scale.squeeze(-1), v, causal=True)
    assert oracle.rel_l1(fp16pv, ref) <= oracle.rel_l1(out, ref) + 1e-4
