"""GPU parity of the int8-QK prefill forward (every backend: the two tensor-memory kernels -- TC = 128 x 64
tiles, two blocks per SM; TC2Q = two 128-row query tiles per block, 128-key tiles -- and mma.sync), through the C ABI.

Bars: int32 logits bit-exact; outputs inside the reference's int8 gate against the fp32
oracle (cos >= 0.999, rel-L1 <= 0.02, SQNR >= 20 dB; reference tests/tolerances.py:74-88) and,
on identical int8 inputs, within cos >= 0.99999 / rel-L1 <= 3e-3 (fp16) or cos >= 0.9999 / rel-L1 <= 1.2e-2 (bf16: P is
rounded to bf16 for the tensor-core P.V) of the CPU restatement and of the reference's own kernel."""

import pytest
import torch

import superl8_b200 as s8
from gpu_helpers import quantized_inputs, ref_fwd, ref_lib
from oracle import oracle
from superl8_b200 import _C, _lib

pytestmark = pytest.mark.gpu

TC, MMA, TC2Q = _lib.SL8_BACKEND_TCGEN05, _lib.SL8_BACKEND_MMA, _lib.SL8_BACKEND_TCGEN05_2Q

# (B, Hq, Hkv, M, N, D, causal)
SHAPES = [
    (1, 2, 2, 128, 128, 128, False), (1, 2, 2, 128, 128, 128, True), (2, 4, 2, 257, 257, 64, True),
    (1, 8, 2, 333, 333, 128, False), (1, 16, 1, 200, 200, 64, False), (1, 2, 1, 100, 300, 128, True),
    (1, 2, 2, 300, 100, 128, True), (1, 4, 4, 64, 1000, 256, False), (1, 2, 2, 384, 384, 256, True),
    (2, 8, 2, 1024, 1024, 128, True), (1, 2, 2, 1, 500, 128, False), (1, 4, 2, 130, 7, 64, True),
]
ODD_D = [(1, 2, 2, 150, 150, 32, True), (1, 4, 2, 200, 200, 72, False), (1, 2, 1, 130, 130, 80, True)]


def run(d, causal, backend, window=-1, want_lse=False, **kw):
    dev = d["dev"]
    if want_lse:
        return _C.attn_int8_fwd_train(dev["q_i8"], dev["q_scale"], dev["k_i8"], dev["k_scale"], dev["v"], causal,
                                      backend=backend)
    return _C.attn_int8_fwd(dev["q_i8"], dev["q_scale"], dev["k_i8"], dev["k_scale"], dev["v"], causal, window,
                            backend=backend, **kw)


def check_against_restatement(out, d, causal, window=-1, rel=3e-3, cos=0.99999):
    rest = oracle.attn_int8_fwd(d["q_i8"], d["q_scale"], d["k_i8"], d["k_scale"], d["v"], causal, window)
    assert torch.isfinite(out.float()).all()
    assert oracle.cos_sim(out, rest) >= cos, oracle.cos_sim(out, rest)
    assert oracle.rel_l1(out, rest) <= rel, oracle.rel_l1(out, rest)


@pytest.mark.parametrize("backend", [TC, MMA, TC2Q])
@pytest.mark.parametrize("B,Hq,Hkv,M,N,D,causal", SHAPES)
def test_fwd_shapes(B, Hq, Hkv, M, N, D, causal, backend, device):
    d = quantized_inputs(10 + D, B, Hq, Hkv, M, D, N=N)
    out = run(d, causal, backend)
    assert out.shape == (B, Hq, M, D) and out.dtype == torch.float16
    assert _C.device_status() == 0
    check_against_restatement(out, d, causal)
    if M == N or not causal:
        oracle.assert_int8_quality(out, oracle.attention_fp32(d["q"], d["k"], d["v"], causal=causal))
    if ref_lib() is not None:
        dev = d["dev"]
        r = ref_fwd(dev["q_i8"], dev["q_scale"], dev["k_i8"], dev["k_scale"], dev["v"], causal)
        assert oracle.cos_sim(out, r) >= 0.99999 and oracle.rel_l1(out, r) <= 3e-3
    assert torch.equal(out, run(d, causal, backend))          # bitwise repeatable


@pytest.mark.parametrize("B,Hq,Hkv,M,N,D,causal", ODD_D)
def test_fwd_odd_head_dims(B, Hq, Hkv, M, N, D, causal, device):
    d = quantized_inputs(20 + D, B, Hq, Hkv, M, D, N=N)
    out = run(d, causal, _lib.SL8_BACKEND_AUTO)
    check_against_restatement(out, d, causal)
    with pytest.raises(RuntimeError, match="not supported"):
        run(d, causal, TC)


@pytest.mark.parametrize("D", [64, 128, 256])
def test_int32_logits_bit_exact(D, device):
    g = torch.Generator().manual_seed(D)
    for M, N in ((128, 128), (200, 333), (1, 129), (385, 64)):
        q = torch.randint(-127, 128, (M, D), generator=g, dtype=torch.int8)
        k = torch.randint(-127, 128, (N, D), generator=g, dtype=torch.int8)
        s = _C.qk_logits_i32(q.to(device), k.to(device))
        assert torch.equal(s.cpu(), oracle.int32_logits(q, k)), (M, N)
    q = torch.full((128, D), -127, dtype=torch.int8)
    k = torch.full((128, D), 127, dtype=torch.int8)
    assert int(_C.qk_logits_i32(q.to(device), k.to(device)).min()) == -127 * 127 * D
    assert _C.device_status() == 0


@pytest.mark.parametrize("backend", [TC, MMA, TC2Q])
def test_bf16_v_and_out(backend, device):
    d = quantized_inputs(31, 1, 4, 2, 300, 128, dtype=torch.bfloat16)
    d["dev"]["v"] = d["dev"]["v"] * 300.0                      # would overflow an fp16 output
    d["v"] = d["v"] * 300.0
    out = run(d, True, backend)
    assert out.dtype == torch.bfloat16
    check_against_restatement(out, d, True, rel=1.2e-2, cos=0.9999)
    dev = d["dev"]
    with pytest.raises(RuntimeError, match="float16 or bfloat16"):
        _C.attn_int8_fwd(dev["q_i8"], dev["q_scale"], dev["k_i8"], dev["k_scale"], dev["v"].float(), True, -1)


def test_bad_head_dim_raises(device):
    q = torch.zeros(1, 2, 64, 96, dtype=torch.int8, device=device)
    sc = torch.ones(1, 2, 64, device=device)
    v = torch.zeros(1, 2, 64, 96, dtype=torch.float16, device=device)
    with pytest.raises(RuntimeError, match="head dim"):
        _C.attn_int8_fwd(q, sc, q, sc, v, False, -1)


@pytest.mark.parametrize("backend", [TC, MMA, TC2Q])
def test_lse(backend, device):
    d = quantized_inputs(32, 1, 4, 2, 200, 128, N=260)
    out, lse = run(d, True, backend, want_lse=True)
    _o, lse_o = oracle.attn_int8_fwd(d["q_i8"], d["q_scale"], d["k_i8"], d["k_scale"], d["v"], True, -1, want_lse=True)
    assert torch.allclose(lse.cpu(), lse_o, rtol=1e-4, atol=1e-4)
    assert torch.equal(out, run(d, True, backend))


@pytest.mark.parametrize("backend", [TC, MMA, TC2Q])
def test_gqa_equals_repeat_interleave_bitwise(backend, device):
    d = quantized_inputs(33, 1, 8, 2, 256, 128)
    out = run(d, True, backend)
    dev = d["dev"]
    k_rep = dev["k_i8"].repeat_interleave(4, dim=1).contiguous()
    ks_rep = dev["k_scale"].repeat_interleave(4, dim=1).contiguous()
    v_rep = dev["v"].repeat_interleave(4, dim=1).contiguous()
    out2 = _C.attn_int8_fwd(dev["q_i8"], dev["q_scale"], k_rep, ks_rep, v_rep, True, -1, backend=backend)
    assert torch.equal(out, out2)


@pytest.mark.parametrize("backend", [TC, MMA, TC2Q])
def test_window(backend, device):
    d = quantized_inputs(34, 1, 4, 2, 400, 128)
    full = run(d, True, backend)
    assert torch.equal(run(d, True, backend, window=400), full)    # window >= S == plain causal
    assert torch.equal(run(d, True, backend, window=100000), full)
    out = run(d, True, backend, window=37)
    check_against_restatement(out, d, True, window=37)
    oracle.assert_int8_quality(out, oracle.attention_fp32(d["q"], d["k"], d["v"], window_left=37))


@pytest.mark.parametrize("backend", [TC, MMA, TC2Q])
def test_fully_masked_rows_are_zero(backend, device):
    # causal with N < M: the first M - N query rows see no key (reference: out 0, lse -inf)
    d = quantized_inputs(35, 1, 2, 2, 300, 128, N=40)
    out, lse = run(d, True, backend, want_lse=True)
    assert float(out[:, :, :260].abs().max()) == 0.0
    assert bool(torch.isinf(lse[:, :, :260]).all())
    check_against_restatement(out, d, True)


@pytest.mark.parametrize("backend", [TC, MMA, TC2Q])
def test_ragged_seqlens(backend, device):
    B, Hq, Hkv, S, D = 4, 4, 1, 512, 64
    d = quantized_inputs(36, B, Hq, Hkv, S, D)
    lens = torch.tensor([512, 100, 257, 1], dtype=torch.int32)
    dev = d["dev"]
    # per-sequence K statistics: quantise each sequence's own slice, as the reference does per call
    k_i8 = torch.zeros_like(d["k_i8"])
    k_scale = torch.zeros_like(d["k_scale"])
    for b in range(B):
        n = int(lens[b])
        _qi, _qs, ki, ks, _ = oracle.quantize_qk(d["q"][b:b + 1, :, :n], d["k"][b:b + 1, :, :n])
        k_i8[b, :, :n], k_scale[b, :, :n] = ki[0], ks[0].squeeze(-1)
    out = _C.attn_int8_fwd(dev["q_i8"], dev["q_scale"], k_i8.to(device), k_scale.to(device), dev["v"], False, -1,
                           seqlens_q=lens.to(device), seqlens_k=lens.to(device), backend=backend)
    ref = oracle.attention_fp32_ragged(d["q"], d["k"], d["v"], lens, lens)
    oracle.assert_int8_quality(out, ref)
    for b in range(B):
        n = int(lens[b])
        assert float(out[b, :, n:].abs().max() if n < S else 0.0) == 0.0
        rest = oracle.attn_int8_fwd(d["q_i8"][b:b + 1, :, :n], d["q_scale"][b:b + 1, :, :n], k_i8[b:b + 1, :, :n],
                                    k_scale[b:b + 1, :, :n], d["v"][b:b + 1, :, :n])
        assert oracle.cos_sim(out[b:b + 1, :, :n], rest) >= 0.99999


def test_python_entry_with_gate_and_smoothing(device):
    # cfg1 of the baseline list: B1 Hq8 Hkv2 S1024 D128 causal
    q, k, v = oracle.make_batch(1, 1, 8, 2, 1024, 128)
    k = k + 0.75                                               # channel offset: K smoothing must remove it
    ref = oracle.attention_fp32(q, k, v, causal=True)
    out = s8.attn_int8_fwd(q.to(device), k.to(device), v.to(device), causal=True)
    assert s8.ops.last_gate_decision is False
    oracle.assert_int8_quality(out, ref)
    # an outlier-dominated Q row demotes the whole call to the full-precision kernel
    q2 = q.clone()
    q2[0, 3, 17, 5] = 70.0
    out2 = s8.attn_int8_fwd(q2.to(device), k.to(device), v.to(device), causal=True)
    assert s8.ops.last_gate_decision is True
    ref2 = oracle.attention_fp32(q2, k, v, causal=True)
    assert oracle.cos_sim(out2, ref2) >= 0.9999 and oracle.rel_l1(out2, ref2) <= 5e-3
    out3 = s8.attn_int8_fwd(q2.to(device), k.to(device), v.to(device), causal=True, internal_accuracy_gate=False)
    assert s8.ops.last_gate_decision is None and torch.isfinite(out3.float()).all()


@pytest.mark.parametrize("D,dtype,backend", [(64, torch.float16, TC), (128, torch.bfloat16, TC), (128, torch.float16, TC),
                                             (256, torch.float16, TC), (128, torch.float16, TC2Q), (128, torch.bfloat16, TC2Q), (80, torch.float16, MMA), (128, torch.float16, MMA),
                                             (64, torch.bfloat16, MMA), (256, torch.float16, MMA)])
def test_fp16_fwd(D, dtype, backend, device):
    q, k, v = oracle.make_batch(40 + D, 2, 4, 2, 300, D, Sk=333, dtype=dtype)
    tol = 5e-3 if dtype == torch.float16 else 2e-2
    for causal, window in ((False, -1), (True, -1), (True, 50)):
        out = _C.attn_fp16_fwd(q.to(device), k.to(device), v.to(device), causal, None, window, None, backend=backend)
        ref = oracle.attention_fp32(q, k, v, causal=causal, window_left=window)
        assert oracle.cos_sim(out, ref) >= 0.9999 and oracle.rel_l1(out, ref) <= tol, (causal, window)
        assert torch.equal(out, _C.attn_fp16_fwd(q.to(device), k.to(device), v.to(device), causal, None, window, None,
                                                 backend=backend))
    assert _C.device_status() == 0
    lens = torch.tensor([300, 77], dtype=torch.int32)
    out = _C.attn_fp16_fwd(q.to(device), k[:, :, :300].contiguous().to(device), v[:, :, :300].contiguous().to(device),
                           True, None, -1, None, seqlens_q=lens.to(device), seqlens_k=lens.to(device), backend=backend)
    ref = oracle.attention_fp32_ragged(q, k[:, :, :300], v[:, :, :300], lens, lens, causal=True)
    assert oracle.cos_sim(out, ref) >= 0.9999 and float(out[1, :, 77:].abs().max()) == 0.0
    if backend == TC:
        with pytest.raises(RuntimeError, match="not supported"):
            qq = torch.zeros(1, 2, 64, 80, dtype=dtype, device=device)
            _C.attn_fp16_fwd(qq, qq, qq, False, None, -1, None, backend=TC)


def test_autograd_wrapper(device):
    q, k, v = (t.to(device).requires_grad_(True) for t in oracle.make_batch(45, 1, 4, 2, 96, 64))
    out = s8.attn(q, k, v, causal=True)
    out.float().square().sum().backward()
    qr, kr, vr = (t.detach().float().requires_grad_(True) for t in (q, k, v))
    kk, vv = kr.repeat_interleave(2, 1), vr.repeat_interleave(2, 1)
    s = torch.einsum("bhmd,bhnd->bhmn", qr, kk) / 8.0
    s = s.masked_fill(~torch.ones(96, 96, dtype=torch.bool, device=device).tril(), float("-inf"))
    ref = torch.softmax(s, -1) @ vv
    ref.square().sum().backward()
    for a, b in ((q.grad, qr.grad), (k.grad, kr.grad), (v.grad, vr.grad)):
        assert oracle.cos_sim(a, b) >= 0.99


def test_full_size_properties_cfg2(device):
    # cfg2: B1 Hq32 Hkv8 S4096 D128 causal.  Too large for the CPU oracle in seconds, so use
    # properties: rows of P sum to 1 (V = ones -> out = 1) and linearity in V.
    B, Hq, Hkv, S, D = 1, 32, 8, 4096, 128
    g = torch.Generator().manual_seed(2002)
    q = torch.randn(B, Hq, S, D, generator=g).half().to(device)
    k = torch.randn(B, Hkv, S, D, generator=g).half().to(device)
    v1 = torch.randn(B, Hkv, S, D, generator=g).half().to(device)
    v2 = torch.randn(B, Hkv, S, D, generator=g).half().to(device)
    ones = torch.ones_like(v1)
    o1 = s8.attn_int8_fwd(q, k, ones, causal=True)
    assert float((o1.float() - 1.0).abs().max()) <= 2e-3
    oa = s8.attn_int8_fwd(q, k, v1, causal=True).float()
    ob = s8.attn_int8_fwd(q, k, v2, causal=True).float()
    oab = s8.attn_int8_fwd(q, k, (v1.float() + v2.float()).half(), causal=True).float()
    assert oracle.rel_l1(oab.cpu(), (oa + ob).cpu()) <= 5e-3
    # first query row attends only key 0 -> equals v[0]
    assert torch.allclose(oa[:, :, 0].cpu(), v1.float().repeat_interleave(4, 1)[:, :, 0].cpu(), atol=2e-3)
    assert _C.device_status() == 0


def test_tensor_peak_probe_runs(device):
    i8 = _C.tensor_peak(True, 512)
    f16 = _C.tensor_peak(False, 512)
    assert _C.device_status() == 0
    assert i8 > f16 > 100.0          # int8 issues at twice the fp16 rate; both far above any CUDA-core figure


@pytest.mark.parametrize("D,dtype", [(128, torch.float16), (64, torch.bfloat16), (256, torch.float16)])
def test_additive_mask_on_the_tensor_memory_kernel(D, dtype, device):
    """The bias is added by the tensor-memory kernel itself (not a detour through the mma.sync kernel):
    both kernels against the fp32 oracle and against each other, for the layouts a caller can hand
    over -- contiguous (one 16-byte load per eight keys), a row pitch that breaks the alignment, a
    transposed view (element by element), broadcast axes -- and with seqlens."""
    B, Hq, Hkv, M, N = 2, 4, 2, 200, 333
    q, k, v = (t.to(device) for t in oracle.make_batch(148, B, Hq, Hkv, M, D, Sk=N, dtype=dtype))
    g = torch.Generator().manual_seed(19)
    tol = 5e-3 if dtype == torch.float16 else 2e-2
    base = (torch.randn(B, Hq, M, N + 3, generator=g) * 2.0).to(dtype)
    base[..., ::7, 3::11] = float("-inf")
    base[0, 1, 5, :] = float("-inf")                         # a row that sees nothing
    layouts = {
        "contiguous": base[..., :N].contiguous().to(device),
        "pitched (rows not 16-byte aligned)": base.to(device)[..., 1:N + 1],
        "transposed": base[..., :N].transpose(2, 3).contiguous().to(device).transpose(2, 3),
        "broadcast over heads": base[:, :1, :, :N].contiguous().to(device),
        "broadcast over batch and heads": base[:1, :1, :, :N].contiguous().to(device),
    }
    for name, bias in layouts.items():
        for causal in (False, True):
            ref = oracle.attention_fp32(q.cpu(), k.cpu(), v.cpu(), causal=causal, mask=bias.cpu().expand(B, Hq, M, N))
            ref = torch.nan_to_num(ref, nan=0.0)     # torch's softmax of a row of -inf is NaN; the kernels write 0 (l == 0)
            tc = _C.attn_fp16_fwd(q, k, v, causal, None, -1, bias, backend=_lib.SL8_BACKEND_TCGEN05)
            mma = _C.attn_fp16_fwd(q, k, v, causal, None, -1, bias, backend=_lib.SL8_BACKEND_MMA)
            assert oracle.cos_sim(tc, ref) >= 0.9999 and oracle.rel_l1(tc, ref) <= tol, (name, causal)
            assert oracle.cos_sim(tc, mma) >= 0.99999 and oracle.rel_l1(tc, mma) <= tol / 2, (name, causal)
            assert torch.equal(tc, _C.attn_fp16_fwd(q, k, v, causal, None, -1, bias)), "the default backend where it serves"
    # the row whose bias is -inf everywhere comes out as zeros
    assert float(_C.attn_fp16_fwd(q, k, v, False, None, -1, layouts["contiguous"])[0, 1, 5].float().abs().max()) == 0.0
    # ragged lengths: the bias of padded keys is never read into a valid row
    sq = torch.tensor([150, 200], dtype=torch.int32, device=device)
    sk = torch.tensor([333, 97], dtype=torch.int32, device=device)
    bias = layouts["contiguous"]
    out = _C.attn_fp16_fwd(q, k, v, False, None, -1, bias, seqlens_q=sq, seqlens_k=sk, backend=_lib.SL8_BACKEND_TCGEN05)
    for bi in range(B):
        mq, nk = int(sq[bi]), int(sk[bi])
        ref = oracle.attention_fp32(q[bi:bi + 1, :, :mq].cpu(), k[bi:bi + 1, :, :nk].cpu(), v[bi:bi + 1, :, :nk].cpu(),
                                    mask=bias[bi:bi + 1, :, :mq, :nk].cpu())
        assert oracle.cos_sim(out[bi:bi + 1, :, :mq], torch.nan_to_num(ref, nan=0.0)) >= 0.9999
    assert _C.device_status(device) == 0


@pytest.mark.parametrize("D,dtype", [(128, torch.float16), (64, torch.bfloat16), (80, torch.float16)])
def test_fp16_fwd_additive_mask(D, dtype, device):
    B, Hq, Hkv, M, N = 2, 4, 2, 150, 200
    q, k, v = oracle.make_batch(48, B, Hq, Hkv, M, D, Sk=N, dtype=dtype)
    g = torch.Generator().manual_seed(9)
    tol = 5e-3 if dtype == torch.float16 else 2e-2
    for shape in ((B, 1, M, N), (1, Hq, M, N), (1, 1, M, N), (B, Hq, M, N)):
        bias = (torch.randn(*shape, generator=g) * 2.0).to(dtype)
        bias[..., ::7, 3::11] = float("-inf")                # some keys hidden from some rows
        for causal in (False, True):
            out = _C.attn_fp16_fwd(q.to(device), k.to(device), v.to(device), causal, None, -1, bias.to(device))
            ref = oracle.attention_fp32(q, k, v, causal=causal, mask=bias)
            assert oracle.cos_sim(out, ref) >= 0.9999 and oracle.rel_l1(out, ref) <= tol, (shape, causal)
    # a broadcast VIEW is indexed in place through its strides
    base = (torch.randn(B, 1, M, N, generator=g)).to(dtype).to(device)
    view = base.expand(B, Hq, M, N)
    out = s8.attn_fp16_fwd(q.to(device), k.to(device), v.to(device), mask=view)
    ref = oracle.attention_fp32(q, k, v, mask=base.cpu())
    assert oracle.cos_sim(out, ref) >= 0.9999
    with pytest.raises(RuntimeError, match="mask"):
        _C.attn_fp16_fwd(q.to(device), k.to(device), v.to(device), False, None, -1, base[:, :, :, :5])


def test_host_buffer_entry_point_equals_the_device_one(device):
    # pinned host tensors in, pinned host tensor out, chunks of the batch on three streams
    q, k, v = oracle.make_batch(77, 5, 4, 2, 200, 64)
    ref = s8.attn_int8_fwd(q.to(device), k.to(device), v.to(device), causal=True).cpu()
    hq, hk, hv = (t.pin_memory() for t in (q, k, v))
    for chunk in (None, 2, 5, 8):
        out = s8.attn_int8_fwd_host(hq, hk, hv, causal=True, chunk_batch=chunk)
        torch.cuda.synchronize()
        assert out.is_pinned() and torch.equal(out, ref), chunk
    with pytest.raises(RuntimeError, match="host tensors"):
        s8.attn_int8_fwd_host(q.to(device), hk, hv)
    # the in-library pipeline (sl8_attn_int8_fwd_host): chunks of one KV head, two to four staging slots,
    # per-chunk gate flags; a chunk with an outlier row is demoted on the device, the others are not
    q2 = q.clone()
    q2[3, 2, 17, 5] = 70.0                                  # batch 3, query head 2 -> KV head 1
    hq2 = q2.pin_memory()
    for kvc, slots in ((1, 2), (1, 4), (2, 3)):
        flags = torch.full((16,), -1, dtype=torch.int32).pin_memory()
        out = s8.attn_int8_fwd_host(hq2, hk, hv, causal=True, kv_heads_per_chunk=kvc, staging_slots=slots, gate_flags=flags)
        torch.cuda.synchronize()
        n_chunks = 5 * (2 // kvc)
        hit = 3 * (2 // kvc) + (1 if kvc == 1 else 0)
        assert [int(f != 0) for f in flags[:n_chunks]] == [int(i == hit) for i in range(n_chunks)], (kvc, flags)
        assert torch.equal(out[:3], ref[:3]) and torch.equal(out[4:], ref[4:])
        full = oracle.attention_fp32(q2[3:4], k[3:4], v[3:4], causal=True)
        sel = slice(0, 4) if kvc == 2 else slice(2, 4)       # the demoted chunk: full-precision bar
        assert oracle.cos_sim(out[3:4, sel], full[:, sel]) >= 0.9999
    assert _C.device_status() == 0


def test_negative_softmax_scale_takes_the_warp_level_kernel(device):
    # the tensor-memory kernel takes row maxima before scaling (wants scale >= 0); the public entry
    # routes a negative scale to the mma.sync backend instead of returning a wrong answer
    q, k, v = oracle.make_batch(78, 1, 4, 2, 200, 128)
    out = s8.attn_int8_fwd(q.to(device), k.to(device), v.to(device), causal=True, scale=-0.08)
    oracle.assert_int8_quality(out, oracle.attention_fp32(q, k, v, causal=True, scale=-0.08), what="negative scale")
