"""The adversarial and behavioural cases of the reference's own forward tests, re-expressed
against this library (reference tests/test_attn_fwd.py:55-113, tests/test_rotation.py,
tests/test_cuda_capture_guard.py).  Gate: the reference's int8 quality bar."""

from unittest import mock

import pytest
import torch

import superl8_b200 as s8
from oracle import oracle
from superl8_b200 import _C, quant


def _qkv(shape_q, seed, hkv=None, device="cuda"):
    g = torch.Generator().manual_seed(seed)
    B, H, S, D = shape_q
    q = torch.randn(B, H, S, D, generator=g).half()
    k = torch.randn(B, hkv or H, S, D, generator=g).half()
    v = torch.randn(B, hkv or H, S, D, generator=g).half()
    return q, k, v


@pytest.mark.gpu
def test_k_channel_outlier_is_absorbed_by_smoothing(device):
    q, k, v = _qkv((2, 4, 512, 64), 1)
    k[..., 13] += 8.0
    out = s8.attn_int8_fwd(q.to(device), k.to(device), v.to(device))
    oracle.assert_int8_quality(out, oracle.attention_fp32(q, k, v), what="outlier-K")


@pytest.mark.gpu
def test_peaked_near_tie_softmax(device):
    g = torch.Generator().manual_seed(2)
    q = torch.randn(1, 4, 256, 64, generator=g).half()
    k = (torch.randn(1, 4, 256, 64, generator=g) * 0.1).half()
    v = torch.randn(1, 4, 256, 64, generator=g).half()
    k[:, :, 0] += 4.0
    k[:, :, 1] += 3.98
    out = s8.attn_int8_fwd(q.to(device), k.to(device), v.to(device))
    oracle.assert_int8_quality(out, oracle.attention_fp32(q, k, v), what="near-tie softmax")


@pytest.mark.gpu
def test_external_gate_bypasses_internal_detector_and_rotation_keeps_quality(device, monkeypatch):
    q, k, v = _qkv((1, 4, 257, 128), 3)

    def must_not_run(*a, **kw):
        raise AssertionError("internal detector ran despite internal_accuracy_gate=False")

    monkeypatch.setattr(quant, "detect_q_outlier_domination", must_not_run)
    out = s8.attn_int8_fwd(q.to(device), k.to(device), v.to(device), rotate=True, internal_accuracy_gate=False)
    assert s8.ops.last_gate_decision is None
    oracle.assert_int8_quality(out, oracle.attention_fp32(q, k, v), what="rotated, externally gated")
    # the rotation is orthonormal: rotating twice with H/sqrt(d) gives the input back
    x = q.to(device)
    assert torch.allclose(quant.rotate_last(quant.rotate_last(x)).float(), x.float(), atol=2e-3)


@pytest.mark.gpu
def test_deterministic_and_finite(device):
    q, k, v = _qkv((2, 4, 512, 64), 4)
    r0 = s8.attn_int8_fwd(q.to(device), k.to(device), v.to(device))
    assert torch.isfinite(r0.float()).all()
    for _ in range(3):
        assert torch.equal(s8.attn_int8_fwd(q.to(device), k.to(device), v.to(device)), r0)


def _outlier_dominated_q():
    q = torch.ones(1, 2, 4, 16, dtype=torch.float16)
    q[..., 3] = 100.0
    return q


def test_gate_is_skipped_during_capture_without_touching_the_tensor():
    """CPU: while a stream is capturing the gate answers False and performs no tensor work
    (its answer needs a device->host read)."""

    class Untouchable(torch.Tensor):
        @classmethod
        def __torch_function__(cls, func, types, args=(), kwargs=None):
            raise AssertionError(f"gate touched q during capture: {func}")

    q = _outlier_dominated_q().as_subclass(Untouchable)
    with mock.patch("torch.cuda.is_current_stream_capturing", return_value=True):
        assert s8.detect_q_outlier_domination(q) is False


@pytest.mark.gpu
def test_gate_fires_outside_capture(device):
    with mock.patch("torch.cuda.is_current_stream_capturing", return_value=False):
        assert s8.detect_q_outlier_domination(_outlier_dominated_q().to(device)) is True
        assert s8.detect_q_outlier_domination(torch.ones(1, 2, 4, 16, dtype=torch.float16, device=device)) is False


@pytest.mark.gpu
def test_int8_path_can_be_captured_in_a_cuda_graph(device):
    q, k, v = (t.to(device) for t in _qkv((1, 4, 256, 128), 5, hkv=2))
    eager = s8.attn_int8_fwd(q, k, v, causal=True)
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        s8.attn_int8_fwd(q, k, v, causal=True)          # warm-up on the side stream
    torch.cuda.current_stream().wait_stream(s)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        out = s8.attn_int8_fwd(q, k, v, causal=True)     # gate skipped while capturing
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(out, eager)


@pytest.mark.gpu
@pytest.mark.parametrize("D", [64, 128])
def test_device_side_gate_matches_the_host_side_gate(device, D):
    """internal_accuracy_gate="device": both kernels are launched and the flag decides on the GPU
    which one works.  Same bits as the host-side gate, on inputs that pass the gate and on inputs
    that trip it."""
    q, k, v = (t.to(device) for t in _qkv((2, 4, 300, D), 11, hkv=2))
    for trip in (False, True):
        if trip:
            q = q.clone()
            q[:, :, :, 3] *= 40.0           # one dominant channel in every row: max / median > 12
        host = s8.attn_int8_fwd(q, k, v, causal=True)
        assert s8.ops.last_gate_decision is trip
        dev = s8.attn_int8_fwd(q, k, v, causal=True, internal_accuracy_gate="device")
        assert s8.ops.last_gate_decision is None and bool(s8.ops.last_gate_flag.item()) is trip
        assert torch.equal(dev, host)
    assert _C.device_status() == 0


@pytest.mark.gpu
def test_gated_call_can_be_captured_with_the_device_side_gate(device):
    """The reference skips its gate under CUDA-graph capture (a host read-back cannot be captured);
    with the decision on the device the gate stays active inside the graph: one captured graph
    serves inputs that pass and inputs that trip the gate."""
    q, k, v = (t.to(device) for t in _qkv((1, 4, 256, 128), 5, hkv=2))
    q_ok, q_bad = q.clone(), q.clone()
    q_bad[:, :, :, 7] *= 40.0
    want_ok = s8.attn_int8_fwd(q_ok, k, v, causal=True)
    assert s8.ops.last_gate_decision is False
    want_bad = s8.attn_int8_fwd(q_bad, k, v, causal=True)
    assert s8.ops.last_gate_decision is True
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        s8.attn_int8_fwd(q, k, v, causal=True, internal_accuracy_gate="device")     # warm-up on the side stream
    torch.cuda.current_stream().wait_stream(s)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        out = s8.attn_int8_fwd(q, k, v, causal=True, internal_accuracy_gate="device")
    for src, want in ((q_ok, want_ok), (q_bad, want_bad), (q_ok, want_ok)):
        q.copy_(src)
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(out, want)
