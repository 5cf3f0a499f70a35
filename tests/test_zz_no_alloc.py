"""The allocation-free decode entry point, called straight through the C ABI.

Some hosts cannot let a library allocate device memory: an application that hands its
plugins a fixed budget, a latency-critical serving loop that keeps the allocator (and the
risk of running out of memory) off its steady-state path, or an engine that manages the
whole device through its own arena.  For them the library keeps the decode's split
partials in a fixed array inside its own image (sl8_attn_int8_decode_static).  This test
checks that variant against the ordinary entry point, which takes a caller workspace,
on two calls in a row (the array is shared and keeps the previous call's contents).
Collected last on purpose: a failure here cannot hide any other test's result.
"""

import ctypes as C

import pytest
import torch

from gpu_helpers import quantized_inputs
from oracle import oracle
from superl8_b200 import _lib

pytestmark = pytest.mark.gpu


def _params(dev, B, Hq, Hkv, N, D, out, ns, lens=None):
    return _lib.DecodeParams(
        q=dev["q_i8"].data_ptr(), q_scale=dev["q_scale"].data_ptr(), k=dev["k_i8"].data_ptr(),
        k_scale=dev["k_scale"].data_ptr(), v=dev["v"].data_ptr(), out=out.data_ptr(),
        context_lens=None if lens is None else lens.data_ptr(), B=B, Hq=Hq, Hkv=Hkv, N=N, D=D, num_splits=ns)


def _with_workspace(lib, p, device):
    nbytes = int(lib.sl8_attn_int8_decode_workspace(C.byref(p)))
    ws = torch.zeros(nbytes, dtype=torch.uint8, device=device)
    rc = lib.sl8_attn_int8_decode(C.byref(p), C.c_void_p(ws.data_ptr()), nbytes, None)
    assert rc == 0, _lib.status_string(rc)
    torch.cuda.synchronize()
    assert lib.sl8_read_device_status(C.c_void_p(ws.data_ptr()), None) == 0


def test_static_scratch_decode_matches_workspace_decode(device):
    lib = _lib.load()
    torch.cuda.set_device(device)
    status = torch.zeros(1, dtype=torch.int32, device=device)
    # two different problems back to back: the second call meets the first call's leftovers
    cases = [(2, 16, 2, 1500, 128, 4, None), (3, 8, 8, 700, 64, -1, torch.tensor([700, 33, 256], dtype=torch.int32))]
    for rep in range(2):
        for (B, Hq, Hkv, N, D, ns, lens) in cases:
            d = quantized_inputs(70 + D, B, Hq, Hkv, 1, D, N=N)
            dev = d["dev"]
            ldev = None if lens is None else lens.to(device)
            out_ws = torch.empty(B, Hq, 1, D, dtype=torch.float16, device=device)
            out_st = torch.full((B, Hq, 1, D), float("nan"), dtype=torch.float16, device=device)
            _with_workspace(lib, _params(dev, B, Hq, Hkv, N, D, out_ws, ns, ldev), device)
            p = _params(dev, B, Hq, Hkv, N, D, out_st, ns, ldev)
            rc = lib.sl8_attn_int8_decode_static(C.byref(p), C.c_void_p(status.data_ptr()), None)
            assert rc == 0, _lib.status_string(rc)
            torch.cuda.synchronize()
            assert int(status.item()) == 0
            if rep == 1:
                # without a caller status word the built-in one is used: zeroed by the call, read here
                out_st2 = torch.full_like(out_st, float("nan"))
                p2 = _params(dev, B, Hq, Hkv, N, D, out_st2, ns, ldev)
                assert lib.sl8_attn_int8_decode_static(C.byref(p2), None, None) == 0
                assert lib.sl8_decode_static_status(None) == 0
                assert torch.equal(out_st2, out_st)
            # same kernels, same split count -> the tolerance of the decode tests holds with room to spare
            assert torch.isfinite(out_st.float()).all()
            assert oracle.cos_sim(out_st, out_ws) >= 0.99999 and oracle.rel_l1(out_st, out_ws) <= 3e-3
            rest = oracle.attn_int8_decode(d["q_i8"], d["q_scale"], d["k_i8"], d["k_scale"], d["v"], 1, lens)
            assert oracle.cos_sim(out_st, rest) >= 0.99999 and oracle.rel_l1(out_st, rest) <= 3e-3


def test_static_scratch_capacity_is_enforced(device):
    lib = _lib.load()
    torch.cuda.set_device(device)
    B, Hq, Hkv, N, D = 8, 64, 8, 4096, 128
    d = quantized_inputs(77, 1, Hq, Hkv, 1, D, N=256)      # pointers only need to be valid and aligned
    dev = d["dev"]
    out = torch.empty(B, Hq, 1, D, dtype=torch.float16, device=device)
    need = 256 + 256 * B * Hq * (D + 2) * 4
    assert need > _lib.DECODE_STATIC_SCRATCH_BYTES
    p = _params(dev, B, Hq, Hkv, N, D, out, 256)
    rc = lib.sl8_attn_int8_decode_static(C.byref(p), None, None)
    assert rc == _lib.ERR_TOO_LARGE and "capacity" in _lib.status_string(rc)
