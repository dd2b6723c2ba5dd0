"""The textual kapy IR reader and the lifting of parsed kernels.

The fixtures under tests/golden/kernels/ are kernels written for this test in
the reference's assembly syntax; tests/golden/ref_inputs/ holds the three kernel
inputs of the reference's own test suite, which are parsed, lifted and run on
the GPU unchanged."""
import glob
import os

import numpy as np
import pytest
import torch

from fake_handle import FakeHandle
from util import bits, normal

HERE = os.path.dirname(os.path.abspath(__file__))
KERNELS = os.path.join(HERE, "golden", "kernels")
# the reference's own test inputs (test/Conversion/KapyToKgpu/*.mlir), unchanged
REF = os.path.join(HERE, "golden", "ref_inputs")


def load(pkg, name):
    mod = pkg.ir.parse_mlir_module(os.path.join(KERNELS, name), pkg.ir.MLIRContext())
    return mod, next(iter(mod.functions.values()))


def test_parse_fixtures(pkg):
    for f in sorted(glob.glob(os.path.join(KERNELS, "*.mlir"))):
        mod = pkg.mlir_text.parse_file(f)
        assert len(mod.functions) == 1 and mod.get_int_attr("kapy.num_warps") >= 1
    with pytest.raises(RuntimeError, match="parse mlir module file failed"):
        pkg.ir.parse_mlir_module(os.path.join(KERNELS, "missing.mlir"), None)
    with pytest.raises(SyntaxError, match="outside the recognised subset"):
        pkg.mlir_text.parse_text("module {\n kapy.func public @f() {\n  gpu.barrier\n }\n}\n")


def test_lift_scale_shift(pkg):
    mod, fn = load(pkg, "scale_shift_bf16.mlir")
    n = 4096
    x, y = torch.zeros(n, dtype=torch.bfloat16), torch.zeros(n, dtype=torch.bfloat16)
    h = FakeHandle()
    pkg.executor.launch(fn, (4, 1, 1), [x, y, n], h, module=mod)
    kind, insts, tin, tout = h.log[0]
    A = pkg.abi
    assert kind == "elementwise" and (tout.size0, tout.size1) == (1, 4096)
    assert [t[0] for t in insts] == [A.OP_LOAD, A.OP_CVT, A.OP_CONST, A.OP_CONST, A.OP_FMA,
                                     A.OP_CVT, A.OP_STORE]


def test_lift_leaky_relu_select(pkg):
    """arith.cmpf feeding arith.select over register tensors becomes part of the
    elementwise program (KAPYB_OP_CMP / KAPYB_OP_SELECT)."""
    mod, fn = load(pkg, "leaky_relu_f32.mlir")
    n = 2048
    x, y = torch.zeros(n), torch.zeros(n)
    h = FakeHandle()
    pkg.executor.launch(fn, (n // 512, 1, 1), [x, y, n], h, module=mod)
    kind, insts, tin, tout = h.log[0]
    A = pkg.abi
    ops = [t[0] for t in insts]
    assert kind == "elementwise" and (tout.size0, tout.size1) == (1, n)
    assert ops.count(A.OP_CMP) == 1 and ops.count(A.OP_SELECT) == 1 and ops[-1] == A.OP_STORE
    cmp_inst = insts[ops.index(A.OP_CMP)]
    assert cmp_inst[1] == A.I1 and cmp_inst[7] == A.CMP_PREDICATES.index("ogt")


def test_lift_row_max(pkg):
    mod, fn = load(pkg, "row_max_f32.mlir")
    m = 64
    src, dst = torch.zeros((m, 128)), torch.zeros((m, 1))
    h = FakeHandle()
    pkg.executor.launch(fn, (m // 8, 1, 1), [src, dst, m], h, module=mod)
    kind, tsrc, tdst, axis, comb = h.log[0]
    assert kind == "reduce" and axis == 1 and comb == pkg.abi.RED_MAX
    assert (tsrc.size0, tsrc.size1, tsrc.stride0) == (64, 128, 128)
    assert (tdst.size0, tdst.size1) == (64, 1)


def test_lift_gemm_ring(pkg):
    mod, fn = load(pkg, "gemm_ring_bf16.mlir")
    M, K, N = 128, 64, 96
    a, b, c = (torch.zeros(s, dtype=torch.bfloat16) for s in ((M, K), (K, N), (M, N)))
    h = FakeHandle()
    pkg.executor.launch(fn, (M // 32, N // 32, 1), [a, b, c, M, K, N], h, module=mod)
    kind, tl, tr, to, ep, way = h.log[0]
    assert kind == "matmul" and way == int(pkg.ir.MatmulImplWay.MMA_M16N8K16_F16)
    assert (tl.size0, tl.size1, tl.stride0, tl.ptr) == (M, K, K, a.data_ptr())
    assert (tr.size0, tr.size1, tr.stride0, tr.ptr) == (K, N, N, b.data_ptr())
    assert (to.size0, to.size1, to.ptr) == (M, N, c.data_ptr())
    assert ep.alpha == 1.0 and ep.rounding == pkg.abi.RN and not ep.bias


def test_lift_gemm_ring_f8_and_tf32(pkg):
    """The same kernel with f8E4M3 x f8E5M2 operands (mma_m16n8k16_f8) and with
    f32 operands (mma_m16n8k8_tf32): element types and impl way reach the call."""
    text = open(os.path.join(KERNELS, "gemm_ring_bf16.mlir")).read()
    body = text.replace("x16xbf16", "x16xf8E4M3").replace("16x32xbf16", "16x32xf8E5M2")
    body = body.replace("[%k, %c1] : !kapy.ptr<1> -> tensor<?x?xbf16", "[%k, %c1] : !kapy.ptr<1> -> tensor<?x?xf8E4M3")
    body = body.replace("%gb = kapy.mk_global %pb[%c0] [%k, %n] [%n, %c1] : !kapy.ptr<1> -> tensor<?x?xbf16",
                        "%gb = kapy.mk_global %pb[%c0] [%k, %n] [%n, %c1] : !kapy.ptr<1> -> tensor<?x?xf8E5M2")
    body = body.replace("%ga[%r0 : %r1, %k0 : %k1] : tensor<?x?xbf16", "%ga[%r0 : %r1, %k0 : %k1] : tensor<?x?xf8E4M3")
    body = body.replace("%gb[%k0 : %k1, %q0 : %q1] : tensor<?x?xbf16", "%gb[%k0 : %k1, %q0 : %q1] : tensor<?x?xf8E5M2")
    body = body.replace("mma_m16n8k16_f16", "mma_m16n8k16_f8")
    M, K, N = 128, 64, 96
    for src, ta, tb, way in ((body, torch.float8_e4m3fn, torch.float8_e5m2, "MMA_M16N8K16_F8"),
                             (text.replace("x16xbf16", "x16xf32").replace("16x32xbf16", "16x32xf32")
                                  .replace("mma_m16n8k16_f16", "mma_m16n8k8_tf32")
                                  .replace("[%k, %c1] : !kapy.ptr<1> -> tensor<?x?xbf16", "[%k, %c1] : !kapy.ptr<1> -> tensor<?x?xf32")
                                  .replace("%gb = kapy.mk_global %pb[%c0] [%k, %n] [%n, %c1] : !kapy.ptr<1> -> tensor<?x?xbf16",
                                           "%gb = kapy.mk_global %pb[%c0] [%k, %n] [%n, %c1] : !kapy.ptr<1> -> tensor<?x?xf32")
                                  .replace("%ga[%r0 : %r1, %k0 : %k1] : tensor<?x?xbf16", "%ga[%r0 : %r1, %k0 : %k1] : tensor<?x?xf32")
                                  .replace("%gb[%k0 : %k1, %q0 : %q1] : tensor<?x?xbf16", "%gb[%k0 : %k1, %q0 : %q1] : tensor<?x?xf32"),
                              torch.float32, torch.float32, "MMA_M16N8K8_TF32")):
        mod = pkg.mlir_text.parse_text(src)
        fn = next(iter(mod.functions.values()))
        a = torch.zeros((M, K)).to(ta)
        b = torch.zeros((K, N)).to(tb)
        c = torch.zeros((M, N), dtype=torch.bfloat16)
        h = FakeHandle()
        pkg.executor.launch(fn, (M // 32, N // 32, 1), [a, b, c, M, K, N], h, module=mod)
        kind, tl, tr, to, ep, got_way = h.log[0]
        assert kind == "matmul" and got_way == int(getattr(pkg.ir.MatmulImplWay, way))
        assert (tl.dtype, tr.dtype, to.dtype) == (pkg.runtime.dtype_code(ta), pkg.runtime.dtype_code(tb),
                                                  pkg.abi.BF16)
        assert (tl.size0, tl.size1, tl.stride0) == (M, K, K) and (tr.size0, tr.size1) == (K, N)


def test_reference_inputs_parse_and_lift(pkg):
    """elementwise_add.mlir, reduce_sum.mlir and matmul.mlir run unchanged: each
    becomes one library call over the region its grid covers."""
    mod = pkg.mlir_text.parse_file(os.path.join(REF, "elementwise_add.mlir"))
    n = 2048
    t = [torch.zeros(n, dtype=torch.float16) for _ in range(3)]
    h = FakeHandle()
    pkg.executor.launch(mod, (n // 512, 1, 1), [*t, n], h)
    kind, insts, tin, tout = h.log[0]
    A = pkg.abi
    assert kind == "elementwise" and [i[0] for i in insts] == [A.OP_LOAD, A.OP_LOAD, A.OP_ADD, A.OP_STORE]
    assert tout.size1 == n and tout.ptr == t[2].data_ptr() and len(tin) == 2

    mod = pkg.mlir_text.parse_file(os.path.join(REF, "reduce_sum.mlir"))
    rows = 64
    src, dst = torch.zeros((rows, 256), dtype=torch.float16), torch.zeros(rows, dtype=torch.float16)
    h = FakeHandle()
    pkg.executor.launch(mod, (rows // 4, 1, 1), [src, dst, rows], h)
    kind, tsrc, tdst, axis, comb = h.log[0]
    assert kind == "reduce" and axis == 1 and comb == A.RED_ADD and tsrc.size0 == rows

    mod = pkg.mlir_text.parse_file(os.path.join(REF, "matmul.mlir"))
    M, K, N = 256, 192, 384
    a, b, c = (torch.zeros(s, dtype=torch.float16) for s in ((M, K), (K, N), (M, N)))
    h = FakeHandle()
    pkg.executor.launch(mod, (M // 128, N // 128, 1), [a, b, c, M, K, N], h)
    kind, tl, tr, to, ep, way = h.log[0]
    assert kind == "matmul" and (tl.size0, tl.size1, tr.size1) == (M, K, N)
    assert (to.size0, to.size1) == (M, N) and way == 1


@pytest.mark.gpu
def test_reference_inputs_run_on_gpu(handle, ko, pkg):
    """The reference's three kernels, launched on the grids their tile sizes
    imply, on seeded data, against the CPU checker."""
    # elementwise_add.mlir:9-25: z = x + y in f16, one program per 512 elements
    mod = pkg.mlir_text.parse_file(os.path.join(REF, "elementwise_add.mlir"))
    n = 512 * 41
    x, y = normal((n,), 21, dtype=torch.float16), normal((n,), 22, dtype=torch.float16)
    zd = torch.zeros(n, dtype=torch.float16, device="cuda")
    ran = pkg.executor.launch(mod, (n // 512, 1, 1), [x.cuda(), y.cuda(), zd, n], handle)
    handle.check()
    assert ran == ["elt_binary"]
    want = ko.eltwise(pkg.programs.binary(pkg.abi.OP_ADD, pkg.abi.F16),
                      [bits(x).reshape(1, -1), bits(y).reshape(1, -1)], [0, 0], (1, n), 0)
    assert np.array_equal(bits(zd.cpu()).reshape(1, -1), want)

    # reduce_sum.mlir:10-25: row sums of [rows, 256] f16 with an f16 addf lambda,
    # one program per 4 rows; every addition rounds to f16, in whatever order
    mod = pkg.mlir_text.parse_file(os.path.join(REF, "reduce_sum.mlir"))
    rows = 4 * 50
    src = normal((rows, 256), 23, dtype=torch.float16)
    dst = torch.zeros(rows, dtype=torch.float16, device="cuda")
    ran = pkg.executor.launch(mod, (rows // 4, 1, 1), [src.cuda(), dst, rows], handle)
    handle.check()
    assert ran == ["reduce_rows"]
    ref, ab = ko.reduce_f64(bits(src), 0, 1)
    got = dst.cpu().double().numpy()
    assert np.all(np.abs(got - ref) <= 256 * 2.0 ** -11 * ab + 1e-30)

    # matmul.mlir:1-134: the pipelined f16 GEMM, grid (M/128, N/128), 4 warps
    mod = pkg.mlir_text.parse_file(os.path.join(REF, "matmul.mlir"))
    M, K, N = 512, 768, 640
    A = normal((M, K), 24, K ** -0.5, dtype=torch.float16)
    B = normal((K, N), 25, dtype=torch.float16)
    Cd = torch.zeros((M, N), dtype=torch.float16, device="cuda")
    ran = pkg.executor.launch(mod, (M // 128, N // 128, 1), [A.cuda(), B.cuda(), Cd, M, K, N],
                              handle)
    handle.check()
    assert ran[0].startswith("tcgen05")
    ref = ko.matmul_f64(bits(A), 0, bits(B), 0)
    err, _ = ko.max_rel_err(Cd.cpu().double().numpy(), ref)
    assert err <= 1e-2, err


@pytest.mark.gpu
def test_fixtures_run_on_gpu(handle, ko, pkg):
    # scale + shift, bit-exact
    mod, fn = load(pkg, "scale_shift_bf16.mlir")
    n = 1024 * 33
    x = normal((n,), 5)
    xd, yd = x.cuda(), torch.zeros(n, dtype=torch.bfloat16, device="cuda")
    assert pkg.executor.launch(fn, (33, 1, 1), [xd, yd, n], handle, module=mod) == ["elt_affine"]
    handle.check()
    want = ko.eltwise(pkg.programs.affine(pkg.abi.BF16, 0.5, 0.1), [bits(x).reshape(1, -1)], [1],
                      (1, n), 1)
    assert np.array_equal(bits(yd.cpu()).reshape(1, -1), want)
    # leaky relu through cmpf + select, bit-exact
    mod, fn = load(pkg, "leaky_relu_f32.mlir")
    n = 512 * 19
    x = normal((n,), 9, dtype=torch.float32)
    yd = torch.zeros(n, dtype=torch.float32, device="cuda")
    assert pkg.executor.launch(fn, (19, 1, 1), [x.cuda(), yd, n], handle, module=mod) == ["elt_interp"]
    handle.check()
    assert torch.equal(yd.cpu(), torch.where(x > 0, x, x * torch.tensor(0.1, dtype=torch.float32)))
    # row max, exact
    mod, fn = load(pkg, "row_max_f32.mlir")
    m = 8 * 25
    src = normal((m, 128), 6, dtype=torch.float32)
    dst = torch.zeros((m, 1), dtype=torch.float32, device="cuda")
    pkg.executor.launch(fn, (25, 1, 1), [src.cuda(), dst, m], handle, module=mod)
    handle.check()
    assert torch.equal(dst.cpu().ravel(), src.max(dim=1).values)
    # pipelined gemm -> tcgen05 kernel
    mod, fn = load(pkg, "gemm_ring_bf16.mlir")
    M, K, N = 256, 512, 384
    A, B = normal((M, K), 7, K ** -0.5), normal((K, N), 8)
    Cd = torch.zeros((M, N), dtype=torch.bfloat16, device="cuda")
    ran = pkg.executor.launch(fn, (M // 32, N // 32, 1), [A.cuda(), B.cuda(), Cd, M, K, N], handle,
                              module=mod)
    handle.check()
    assert ran[0].startswith("tcgen05")
    ref = ko.matmul_f64(bits(A), 1, bits(B), 1)
    err, _ = ko.max_rel_err(Cd.cpu().double().numpy(), ref)
    assert err <= 1e-2


def _gemm_with_epilogue(tail: str) -> str:
    """gemm_ring_bf16.mlir with the lines between the loop and the store replaced."""
    text = open(os.path.join(KERNELS, "gemm_ring_bf16.mlir")).read()
    head, rest = text.split("    %out = arith.truncf %acc", 1)
    rest = rest.split("\n", 1)[1]
    return head + tail + rest


def test_lift_matmul_epilogues(pkg):
    """scale, relu and the downcast after the accumulator become the fused
    epilogue; orders the fused epilogue cannot express are refused."""
    M, K, N = 128, 64, 96
    a, b, c = (torch.zeros(s, dtype=torch.bfloat16) for s in ((M, K), (K, N), (M, N)))
    ok = _gemm_with_epilogue(
        "    %half = arith.constant dense<5.000000e-01> : tensor<32x32xf32, #values>\n"
        "    %zero2 = arith.constant dense<0.000000e+00> : tensor<32x32xf32, #values>\n"
        "    %sc = arith.mulf %acc, %half : tensor<32x32xf32, #values>\n"
        "    %re = arith.maximumf %sc, %zero2 : tensor<32x32xf32, #values>\n"
        "    %out = arith.truncf %re : tensor<32x32xf32, #values> to tensor<32x32xbf16, #values>\n")
    mod = pkg.mlir_text.parse_text(ok)
    h = FakeHandle()
    pkg.executor.launch(next(iter(mod.functions.values())), (M // 32, N // 32, 1),
                        [a, b, c, M, K, N], h, module=mod)
    kind, tl, tr, to, ep, way = h.log[0]
    assert kind == "matmul" and ep.alpha == 0.5 and ep.activation == pkg.abi.ACT_RELU
    # relu before the scale: act(alpha * acc) is not alpha * act(acc) in general
    bad = _gemm_with_epilogue(
        "    %half = arith.constant dense<-5.000000e-01> : tensor<32x32xf32, #values>\n"
        "    %zero2 = arith.constant dense<0.000000e+00> : tensor<32x32xf32, #values>\n"
        "    %re = arith.maximumf %acc, %zero2 : tensor<32x32xf32, #values>\n"
        "    %sc = arith.mulf %re, %half : tensor<32x32xf32, #values>\n"
        "    %out = arith.truncf %sc : tensor<32x32xf32, #values> to tensor<32x32xbf16, #values>\n")
    mod = pkg.mlir_text.parse_text(bad)
    with pytest.raises(pkg.executor.Unsupported, match="relu is recognised once"):
        pkg.executor.launch(next(iter(mod.functions.values())), (M // 32, N // 32, 1),
                            [a, b, c, M, K, N], FakeHandle(), module=mod)
