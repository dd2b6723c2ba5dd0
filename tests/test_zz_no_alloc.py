"""kapyb_matmul_decode_static: the decode-shape matmul for callers that cannot
allocate device memory (its split-K scratch is a fixed array inside the
library).  Checked through the C ABI against the ordinary entry point,
kapyb_matmul, on two calls in a row -- the second call finds the array as the
first left it.  Split tiles are summed in arrival order, so the two entry points
agree to the matmul parity tolerance (max relative error 1e-2 against a floor of
2^-6 rms), not bit for bit.

This file sorts last on purpose: a run that stops at the first failure has
already been through every other test.
"""
import ctypes as C

import pytest
import torch

from util import normal, uniform

pytestmark = pytest.mark.gpu


def rel_err(a: torch.Tensor, b: torch.Tensor) -> float:
    a, b = a.double(), b.double()
    tau = b.pow(2).mean().sqrt().item() / 64 or 1e-30
    return ((a - b).abs() / b.abs().clamp_min(tau)).max().item()


def call_static(pkg, lhs, rhs, out, bias=None, sync=1):
    lib = pkg.abi.load()
    tl, tr, to = pkg.tensor2d(lhs), pkg.tensor2d(rhs), pkg.tensor2d(out)
    ep = pkg.abi.Epilogue(1.0, bias.data_ptr() if bias is not None else None,
                          pkg.runtime.dtype_code(bias.dtype) if bias is not None else 2, 1,
                          pkg.abi.ACT_NONE, pkg.abi.RN)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    st = lib.kapyb_matmul_decode_static(C.byref(tl), C.byref(tr), C.byref(to), C.byref(ep), sync,
                                        stream)
    return st, lib.kapyb_last_error_string(None).decode()


@pytest.mark.parametrize("shape", [(16, 3584, 2048), (5, 1000, 520)])
def test_two_calls_match_the_ordinary_entry_point(handle, pkg, shape):
    M, N, K = shape
    torch.cuda.set_device(0)
    X = normal((M, K), 1005).cuda()
    W = normal((K, N), 2005, 0.02).cuda()
    bias = uniform((N,), 15, -0.1, 0.1, torch.bfloat16).cuda()
    want = handle.matmul(X, W, bias=bias)
    handle.check()
    assert handle.last_kernel == "tcgen05_skinny"
    for call in range(2):
        got = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
        st, msg = call_static(pkg, X, W, got, bias=bias)
        assert st == pkg.abi.OK, msg
        torch.cuda.synchronize()
        assert not torch.isnan(got).any(), f"call {call}: output not fully written"
        assert rel_err(got, want) <= 1e-2, f"call {call}"
    # and the ordinary path is undisturbed afterwards
    again = handle.matmul(X, W, bias=bias)
    handle.check()
    assert rel_err(again, want) <= 1e-2


def test_refuses_what_does_not_fit(pkg):
    torch.cuda.set_device(0)
    z = lambda s: torch.zeros(s, dtype=torch.bfloat16, device="cuda")
    # 131200 columns need 1026 tile counters of 16 bytes: beyond the fixed 16 KiB
    st, msg = call_static(pkg, z((1, 64)), z((64, 131200)), z((1, 131200)))
    assert st == pkg.abi.UNSUPPORTED and "fixed scratch" in msg
    st, msg = call_static(pkg, z((65, 64)), z((64, 256)), z((65, 256)))
    assert st == pkg.abi.UNSUPPORTED and "M <= 64" in msg
    st, msg = call_static(pkg, z((8, 64)), z((32, 256)), z((8, 256)))
    assert st == pkg.abi.INVALID_ARG and "columns of lhs" in msg
