"""kapyb_matmul_decode_static: the decode-shape matmul for callers that cannot
allocate device memory (its split-tile scratch is a fixed array inside the
library).  Checked through the C ABI, on two calls in a row -- the second call
finds the array as the first left it -- against both the ordinary entry point,
kapyb_matmul, and the CPU checker.  A tile that is split between SMs is summed
in CTA order, not arrival order, so the two entry points must agree bit for
bit; against the f64 checker the matmul tolerance applies (max relative error
1e-2 over a floor of 2^-6 rms).

This file sorts last on purpose: a run that stops at the first failure has
already been through every other test.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from util import bits, code, normal, uniform

pytestmark = pytest.mark.gpu


def call_static(pkg, lhs, rhs, out, bias=None, bias_axis=1, activation=0, alpha=1.0, sync=1):
    lib = pkg.abi.load()
    tl, tr, to = pkg.tensor2d(lhs), pkg.tensor2d(rhs), pkg.tensor2d(out)
    ep = pkg.abi.Epilogue(alpha, bias.data_ptr() if bias is not None else None,
                          pkg.runtime.dtype_code(bias.dtype) if bias is not None else 2, bias_axis,
                          activation, pkg.abi.RN)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    st = lib.kapyb_matmul_decode_static(C.byref(tl), C.byref(tr), C.byref(to), C.byref(ep), sync,
                                        stream)
    return st, lib.kapyb_last_error_string(None).decode()


def oracle_err(ko, got, X, W, **ep):
    """Max relative error of `got` against the f64 evaluation of the same problem."""
    kw = {}
    if ep.get("bias") is not None:
        kw.update(bias=bits(ep["bias"]), bias_dtype=code(ep["bias"].dtype),
                  bias_axis=ep.get("bias_axis", 1))
    ref = ko.matmul_f64(bits(X), code(X.dtype), bits(W), code(W.dtype), alpha=ep.get("alpha", 1.0),
                        activation=ep.get("activation", 0), **kw)
    err, _ = ko.max_rel_err(ko.from_bits(bits(got), code(got.dtype)), ref)
    return err


@pytest.mark.parametrize("shape", [(16, 3584, 2048), (5, 1000, 520)])
def test_two_calls_match_the_ordinary_entry_point_and_the_checker(handle, pkg, ko, shape):
    M, N, K = shape
    torch.cuda.set_device(0)
    X = normal((M, K), 1005).cuda()
    W = normal((K, N), 2005, 0.02).cuda()
    bias = uniform((N,), 15, -0.1, 0.1, torch.bfloat16).cuda()
    want = handle.matmul(X, W, bias=bias)
    handle.check()
    assert handle.last_kernel == "tcgen05_skinny"
    assert oracle_err(ko, want, X, W, bias=bias) <= 1e-2
    outs = []
    for call in range(2):
        got = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
        st, msg = call_static(pkg, X, W, got, bias=bias)
        assert st == pkg.abi.OK, msg
        torch.cuda.synchronize()
        assert not torch.isnan(got).any(), f"call {call}: output not fully written"
        assert torch.equal(got, want), f"call {call}: differs from kapyb_matmul"
        assert oracle_err(ko, got, X, W, bias=bias) <= 1e-2, f"call {call}"
        outs.append(got)
    assert torch.equal(outs[0], outs[1])
    # and the ordinary path is undisturbed afterwards
    again = handle.matmul(X, W, bias=bias)
    handle.check()
    assert torch.equal(again, want)


def test_other_layouts_and_epilogues(handle, pkg, ko):
    """M-contiguous activations, K-contiguous weights, an f16 problem with a
    per-row bias and a fused activation, an f32 output: each against the checker
    and, bit for bit, against kapyb_matmul."""
    torch.cuda.set_device(0)
    M, N, K = 24, 1408, 1088
    cases = []
    Xt = normal((K, M), 31).cuda().t()                  # [M, K] with unit stride on M
    Wk = normal((N, K), 32, 0.03).cuda().t()            # [K, N] with unit stride on K
    cases.append((Xt, Wk, torch.bfloat16, {}))
    Xh = uniform((M, K), 33).cuda()
    Wh = uniform((K, N), 34, -0.05, 0.05).cuda()
    rb = uniform((M,), 35, -0.5, 0.5, torch.float32).cuda()
    cases.append((Xh, Wh, torch.float16,
                  dict(bias=rb, bias_axis=0, activation=pkg.abi.ACT_GELU_TANH, alpha=0.75)))
    cases.append((Xh, Wh, torch.float32, {}))
    for X, W, odt, ep in cases:
        want = handle.matmul(X, W, out_dtype=odt, **ep)
        handle.check()
        assert handle.last_kernel == "tcgen05_skinny"
        for call in range(2):
            got = torch.full((M, N), float("nan"), dtype=odt, device="cuda")
            st, msg = call_static(pkg, X, W, got, **ep)
            assert st == pkg.abi.OK, msg
            torch.cuda.synchronize()
            assert torch.equal(got, want), (odt, call)
            assert oracle_err(ko, got, X, W, **ep) <= 1e-2, (odt, call)


def test_takes_no_device_memory(pkg):
    """Free device memory as the driver reports it does not move across calls
    (the first call on the device, which resolves the array's address, is made
    before the reading)."""
    torch.cuda.set_device(0)
    X = normal((16, 1024), 41).cuda()
    W = normal((1024, 2048), 42, 0.02).cuda()
    out = torch.empty((16, 2048), dtype=torch.bfloat16, device="cuda")
    st, msg = call_static(pkg, X, W, out)
    assert st == pkg.abi.OK, msg
    torch.cuda.synchronize()
    free0, _ = torch.cuda.mem_get_info()
    for _ in range(5):
        st, msg = call_static(pkg, X, W, out)
        assert st == pkg.abi.OK, msg
    torch.cuda.synchronize()
    free1, _ = torch.cuda.mem_get_info()
    assert free1 == free0, f"free memory moved by {free0 - free1} bytes"


def test_refuses_what_does_not_fit_and_recovers(handle, pkg):
    torch.cuda.set_device(0)
    z = lambda s: torch.zeros(s, dtype=torch.bfloat16, device="cuda")
    st, msg = call_static(pkg, z((65, 64)), z((64, 256)), z((65, 256)))
    assert st == pkg.abi.UNSUPPORTED and "M <= 64" in msg
    st, msg = call_static(pkg, z((8, 64)), z((32, 256)), z((8, 256)))
    assert st == pkg.abi.INVALID_ARG and "columns of lhs" in msg
    # a refused call launches nothing and leaves the array usable
    X = normal((8, 512), 51).cuda()
    W = normal((512, 640), 52, 0.05).cuda()
    want = handle.matmul(X, W)
    handle.check()
    got = torch.empty_like(want)
    st, msg = call_static(pkg, X, W, got)
    assert st == pkg.abi.OK, msg
    torch.cuda.synchronize()
    assert torch.equal(got, want)
    # an unchecked call (sync_and_check = 0) followed by a checked one
    st, msg = call_static(pkg, X, W, got, sync=0)
    assert st == pkg.abi.OK, msg
    st, msg = call_static(pkg, X, W, got, sync=1)
    assert st == pkg.abi.OK, msg
    assert torch.equal(got, want)
