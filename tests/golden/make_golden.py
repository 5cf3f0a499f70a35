"""Generates tests/golden/*.npz by running the REFERENCE's own Python code on CPU.

Run in a container that has the reference checkout (it cannot travel to a GPU box):
    python tests/golden/make_golden.py /path/to/reference [group ...]
Inputs are seeded; inputs and the reference's outputs are both stored so the tests
never need the reference.  16-bit floats are stored as raw bit patterns.
"""

import os
import sys
from pathlib import Path

import numpy as np
import torch

_root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("SUPERL8_REFERENCE_ROOT")
if not _root or not (Path(_root) / "superl8").is_dir():
    sys.exit("usage: python tests/golden/make_golden.py /path/to/reference   (or set SUPERL8_REFERENCE_ROOT)")
ref_root = Path(_root)
sys.path.insert(0, str(ref_root))
sys.path.insert(0, str(ref_root / "tests"))

from superl8.quant.core import (  # noqa: E402
    detect_q_outlier_domination,
    quantize_int8_rowwise,
    quantize_qk,
    smooth_k,
)
import reference as ref_oracles  # noqa: E402  (reference tests/reference.py)
import tolerances as ref_tol  # noqa: E402  (reference tests/tolerances.py)

OUT = Path(__file__).resolve().parent


def bits(t: torch.Tensor) -> np.ndarray:
    if t.dtype in (torch.float16, torch.bfloat16):
        return t.contiguous().view(torch.int16).numpy()
    return t.contiguous().numpy()


def gen(seed):
    return torch.Generator().manual_seed(seed)


def quant_cases():
    out = {}
    cases = {
        "f16_128": (torch.randn(37, 128, generator=gen(1)).half(), "float16"),
        "f16_64": (torch.randn(50, 64, generator=gen(2)).half() * 3.0, "float16"),
        "bf16_128": (torch.randn(33, 128, generator=gen(3)).bfloat16(), "bfloat16"),
        "f32_72": (torch.randn(21, 72, generator=gen(4)), "float32"),
        "f16_odd33": (torch.randn(19, 33, generator=gen(5)).half(), "float16"),
        "f16_256": (torch.randn(17, 256, generator=gen(6)).half() * 0.01, "float16"),
    }
    x = cases["f16_128"][0]
    x[3] = 0                      # zero row -> scale 1
    x[5, 7] = 1000.0              # outlier row
    x[6] = 0
    x[6, 0] = -65504.0            # fp16 max: saturates to -127
    for name, (x, dt) in cases.items():
        q, s = quantize_int8_rowwise(x)      # reference CPU branch
        out[f"{name}__x"] = bits(x)
        out[f"{name}__dtype"] = np.array(dt)
        out[f"{name}__q"] = q.numpy()
        out[f"{name}__scale"] = s.numpy()
    np.savez_compressed(OUT / "quant_rowwise.npz", **out)


def smooth_cases():
    out = {}
    cases = {
        "short": torch.randn(2, 2, 300, 64, generator=gen(11)).half() + 0.5,
        "chunked": torch.randn(1, 1, 2500, 64, generator=gen(12)).half() * 2.0 - 1.0,
        "bf16": (torch.randn(1, 2, 130, 128, generator=gen(13)) + 2.0).bfloat16(),
    }
    for name, k in cases.items():
        k_s, k_mean = smooth_k(k)
        out[f"{name}__k"] = bits(k)
        out[f"{name}__dtype"] = np.array(str(k.dtype).replace("torch.", ""))
        out[f"{name}__k_s"] = bits(k_s)
        out[f"{name}__k_mean"] = k_mean.numpy()
    np.savez_compressed(OUT / "smooth_k.npz", **out)


def gate_cases():
    out = {}
    base = torch.randn(2, 4, 64, 128, generator=gen(21)).half()
    spike = base.clone()
    spike[1, 2, 17, 5] = 60.0
    chan = base.clone()
    chan[:, :, :, 9] *= 20.0
    d64 = torch.randn(1, 2, 512, 64, generator=gen(22)).half()
    near = torch.ones(1, 1, 4, 8).half()
    near[0, 0, 0, 0] = 12.0      # ratio exactly 12 -> not > 12
    near[0, 0, 1, 0] = 12.01     # just above
    near[0, 0, 1, 1:] = 1.0
    for name, q in {"clean": base, "spike": spike, "chan20": chan, "d64": d64, "near": near}.items():
        out[f"{name}__q"] = bits(q)
        out[f"{name}__flag"] = np.array(detect_q_outlier_domination(q))
        qa = q.float().abs()
        out[f"{name}__ratio"] = (qa.amax(-1) / (qa.median(-1).values + 1e-10)).numpy()
    np.savez_compressed(OUT / "outlier_gate.npz", **out)


def qk_cases():
    out = {}
    q = torch.randn(1, 4, 96, 64, generator=gen(31)).half()
    k = torch.randn(1, 2, 80, 64, generator=gen(32)).half() + 0.25
    for name, sc in {"default": None, "scaled": 0.2}.items():
        q_i8, q_scale, k_i8, k_scale, k_mean = quantize_qk(q, k, softmax_scale=sc)
        out[f"{name}__q_i8"] = q_i8.numpy()
        out[f"{name}__q_scale"] = q_scale.numpy()
        out[f"{name}__k_i8"] = k_i8.numpy()
        out[f"{name}__k_scale"] = k_scale.numpy()
        out[f"{name}__k_mean"] = k_mean.numpy()
    out["q"] = bits(q)
    out["k"] = bits(k)
    np.savez_compressed(OUT / "quantize_qk.npz", **out)


def attention_cases():
    out = {}
    g = gen(41)
    q = torch.randn(2, 4, 40, 32, generator=g).half()
    k = torch.randn(2, 2, 56, 32, generator=g).half()
    v = torch.randn(2, 2, 56, 32, generator=g).half()
    out["q"], out["k"], out["v"] = bits(q), bits(k), bits(v)
    out["noncausal"] = ref_oracles.attention_fp32_oracle(q, k, v).numpy()
    out["causal_rect"] = ref_oracles.attention_fp32_oracle(q, k, v, causal=True).numpy()
    out["scaled"] = ref_oracles.attention_fp32_oracle(q, k, v, causal=True, scale=0.3).numpy()
    out["window9"] = ref_oracles.attention_fp32_window_oracle(q, k, v, window_left=9).numpy()
    a = torch.randn(3, 50, generator=g)
    b = a + 0.05 * torch.randn(3, 50, generator=g)
    out["metric_a"], out["metric_b"] = a.numpy(), b.numpy()
    out["metric_vals"] = np.array([ref_tol.cos_sim(b, a), ref_tol.rel_l1(b, a), ref_tol.sqnr_db(b, a)])
    np.savez_compressed(OUT / "attention_fp32.npz", **out)


def backward_cases():
    """Gradients of the reference's own definitions: superl8/autograd.py::_attn_backward for
    equal head counts, and autograd through tests/reference.py::attention_fp32_oracle (the
    check its CUDA-backward tests use, tests/test_attn_bwd_cuda.py:43-46) for grouped heads."""
    from superl8.autograd import _attn_backward

    out = {}
    g = gen(51)

    def fwd_and_lse(q, k, v, causal, scale):
        kf, vf = k.float(), v.float()
        rep = q.shape[1] // k.shape[1]
        if rep > 1:
            kf, vf = kf.repeat_interleave(rep, dim=1), vf.repeat_interleave(rep, dim=1)
        s = torch.einsum("bhmd,bhnd->bhmn", q.float(), kf) * scale
        if causal:
            m, n = s.shape[-2:]
            s = s.masked_fill(~torch.ones(m, n, dtype=torch.bool).tril(n - m), float("-inf"))
        lse = torch.logsumexp(s, dim=-1).float()     # as superl8/ops.py:49-58 recomputes it
        o = torch.einsum("bhmn,bhnd->bhmd", torch.softmax(s, dim=-1), vf).half()
        return o, lse

    cases = {
        "mha": (1, 2, 2, 48, 48, 32, False, 32 ** -0.5),
        "mha_causal": (2, 2, 2, 70, 70, 64, True, 64 ** -0.5),
        "rect_causal": (1, 2, 2, 40, 56, 32, True, 0.25),
        "gqa_causal": (1, 4, 2, 50, 50, 64, True, 64 ** -0.5),
        "mqa": (1, 4, 1, 33, 65, 128, False, 128 ** -0.5),
    }
    for name, (B, Hq, Hkv, M, N, D, causal, scale) in cases.items():
        q = torch.randn(B, Hq, M, D, generator=g).half()
        k = torch.randn(B, Hkv, N, D, generator=g).half()
        v = torch.randn(B, Hkv, N, D, generator=g).half()
        do = torch.randn(B, Hq, M, D, generator=g).half()
        o, lse = fwd_and_lse(q, k, v, causal, scale)
        if Hq == Hkv:
            dq, dk, dv = _attn_backward(q, k, v, o, do, causal, scale)
        else:
            qf, kf, vf = (t.float().requires_grad_(True) for t in (q, k, v))
            ref_oracles.attention_fp32_oracle(qf, kf, vf, causal=causal, scale=scale).backward(do.float())
            dq, dk, dv = qf.grad, kf.grad, vf.grad
        for key, val in dict(q=q, k=k, v=v, o=o, do=do).items():
            out[f"{name}__{key}"] = bits(val)
        out[f"{name}__lse"] = lse.numpy()
        out[f"{name}__dq"], out[f"{name}__dk"], out[f"{name}__dv"] = dq.numpy(), dk.numpy(), dv.numpy()
        out[f"{name}__cfg"] = np.array([int(causal), scale])
    np.savez_compressed(OUT / "attn_backward.npz", **out)


def varlen_cases():
    """Packed-layout K prologue of the reference: superl8/ops.py::_varlen_smooth_k (ragged and
    equal-length branches) followed by its row quantiser."""
    from superl8.ops import _varlen_smooth_k

    out = {}
    g = gen(61)
    for name, lens, H, D in (("ragged", [37, 5, 0, 120, 64], 2, 64), ("equal", [48, 48, 48], 3, 32)):
        cu = torch.tensor([0] + list(np.cumsum(lens)), dtype=torch.int32)
        k = (torch.randn(int(cu[-1]), H, D, generator=g) + 0.3).half()
        k_s = _varlen_smooth_k(k, cu, max(lens))
        k_i8, k_scale = quantize_int8_rowwise(k_s)
        out[f"{name}__k"], out[f"{name}__cu"] = bits(k), cu.numpy()
        out[f"{name}__k_s"], out[f"{name}__k_i8"], out[f"{name}__k_scale"] = bits(k_s), k_i8.numpy(), k_scale.numpy()
    np.savez_compressed(OUT / "varlen_prologue.npz", **out)


def v_cache_cases():
    """Per-channel V quantiser of the reference (superl8/quant/core.py::quantize_v_perchannel)."""
    from superl8.quant.core import quantize_v_perchannel

    out = {}
    g = gen(71)
    cases = {"f16": torch.randn(2, 2, 200, 64, generator=g).half() * 1.7,
             "bf16": (torch.randn(1, 2, 1100, 64, generator=g) * 0.3).bfloat16()}
    cases["f16"][0, 1, :, 5] = 0          # a zero channel -> scale 1
    cases["f16"][1, 0, 17, 9] = 300.0     # an outlier sets its channel's scale
    for name, v in cases.items():
        v_i8, v_scale = quantize_v_perchannel(v)
        out[f"{name}__v"] = bits(v)
        out[f"{name}__dtype"] = np.array(str(v.dtype).replace("torch.", ""))
        out[f"{name}__v_i8"], out[f"{name}__v_scale"] = v_i8.numpy(), v_scale.numpy()
    np.savez_compressed(OUT / "v_perchannel.npz", **out)

def rotation_cases():
    """rotate=True prologue: the Hadamard rotation alone and quantize_qk with it."""
    from superl8.quant.rotation import rotate_last

    out = {}
    for name, x in {"f16_128": torch.randn(9, 128, generator=gen(61)).half() * 2.0,
                    "bf16_64": torch.randn(7, 64, generator=gen(62)).bfloat16(),
                    "f16_32": torch.randn(5, 32, generator=gen(63)).half()}.items():
        out[f"{name}__x"] = bits(x)
        out[f"{name}__rot"] = bits(rotate_last(x))
    q = torch.randn(1, 4, 70, 128, generator=gen(64)).half()
    k = torch.randn(1, 2, 90, 128, generator=gen(65)).half() + 0.5
    k[..., 5] *= 12.0                              # an outlier channel: what the rotation is for
    q_i8, q_scale, k_i8, k_scale, k_mean = quantize_qk(q, k, rotate=True)
    out.update(q=bits(q), k=bits(k), q_i8=q_i8.numpy(), q_scale=q_scale.numpy(), k_i8=k_i8.numpy(),
               k_scale=k_scale.numpy(), k_mean=k_mean.numpy())
    np.savez_compressed(OUT / "rotation.npz", **out)


if __name__ == "__main__":
    torch.set_num_threads(1)
    cases = dict(quant=quant_cases, smooth=smooth_cases, gate=gate_cases, qk=qk_cases, attention=attention_cases,
                 backward=backward_cases, varlen=varlen_cases, v_cache=v_cache_cases, rotation=rotation_cases)
    only = sys.argv[2:]                            # optional: names of the case groups to regenerate
    for name, fn in cases.items():
        if not only or name in only:
            fn()
    for f in sorted(OUT.glob("*.npz")):
        print(f.name, f.stat().st_size)
