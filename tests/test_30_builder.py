"""The Builder shim: same method names as the reference's ir.Builder
(python/src/ir.cc:480-1181), recording a graph that the executor lifts to the C
ABI.  CPU tests check the lifting against a recording handle; GPU tests run the
kernels and compare with the CPU checker."""
import os

import numpy as np
import pytest
import torch

from fake_handle import FakeHandle
from util import bits, normal


def build_affine_gelu(pkg, dt_name="bf16", tile=256, warps=4):
    """y = gelu_tanh(x*0.5 + 0.1) written op by op against the builder surface,
    as a [1, n] tensor cut into [1, tile] tiles per warp."""
    ir = pkg.ir
    b = ir.Builder(ir.MLIRContext())
    mod = b.create_module()
    mod.set_attr("kapy.num_warps", warps)
    ptr, i32 = b.get_pointer_type(1), b.get_int32_type()
    fn = b.get_or_create_function(mod, "gelu_kernel", b.get_function_type([ptr, ptr, i32], []),
                                  "public", False)
    mod.push_back(fn)
    b.set_insertion_point_to_start(fn.add_entry_block())
    x, y, n = fn.get_argument(0), fn.get_argument(1), fn.get_argument(2)
    et = getattr(b, f"get_{'bfloat16' if dt_name == 'bf16' else 'float16'}_type")()
    f32 = b.get_float32_type()
    c0, c1 = b.create_constant_int32(0), b.create_constant_int32(1)
    gx = b.create_mk_global(x, c0, c1, n, n, c1, et)
    gy = b.create_mk_global(y, c0, c1, n, n, c1, et)
    pid, wid = b.create_program_id(0), b.create_warp_id()
    lo = b.create_addi(b.create_muli(pid, b.create_constant_int32(tile * warps)),
                       b.create_muli(wid, b.create_constant_int32(tile)))
    hi = b.create_addi(lo, b.create_constant_int32(tile))
    vx = b.create_sv_global(gx, c0, c1, lo, hi, [1, tile])
    vy = b.create_sv_global(gy, c0, c1, lo, hi, [1, tile])
    t = b.create_ld_global(vx, ir.PaddingOption.ZERO, ir.CacheModifier.NONE,
                           ir.EvictPriority.EVICT_NORMAL, False)
    tf = b.create_extf(b.get_tensor_type([1, tile], f32, ir.MemorySpace.REGISTER_FILE), t)
    splat = lambda v: b.create_splat(b.create_constant_float32(v), [1, tile])
    u = b.create_fma(tf, splat(0.5), splat(0.1))
    t2 = b.create_mulf(b.create_mulf(splat(0.044715), u), u)
    k = b.create_mulf(splat(0.7978845608), b.create_fma(t2, u, u))
    e = b.create_exp(b.create_mulf(splat(-2.0), k))
    yv = b.create_divf(u, b.create_addf(splat(1.0), e))
    out = b.create_truncf(b.get_tensor_type([1, tile], et, ir.MemorySpace.REGISTER_FILE), yv)
    b.create_st_global(out, vy, ir.CacheModifier.NONE, ir.EvictPriority.EVICT_NORMAL, False)
    b.create_return([])
    fn.finalize()
    return mod, fn


def test_builder_surface_matches_reference_names(pkg):
    """Every create_* the path needs exists with the reference's name."""
    b = pkg.ir.Builder(pkg.ir.MLIRContext())
    for name in ["create_mk_global", "create_sv_global", "create_ld_global", "create_st_global",
                 "create_matmul", "create_splat", "create_broadcast", "create_addf", "create_subf",
                 "create_mulf", "create_divf", "create_fma", "create_exp", "create_exp2",
                 "create_erf", "create_sqrt", "create_rsqrt", "create_absf", "create_maximumf",
                 "create_minimumf", "create_maxnumf", "create_minnumf", "create_clampf",
                 "create_extf", "create_truncf", "create_fptofp", "create_reduce",
                 "create_program_id", "create_warp_id", "create_for", "create_yield",
                 "create_return", "get_or_create_function", "create_constant_float32",
                 "get_tensor_type", "get_pointer_type"]:
        assert callable(getattr(b, name)), name
    with pytest.raises(NotImplementedError):
        b.create_elementwise_inline_asm()
    with pytest.raises(IndexError):              # py::index_error in the reference
        b.set_insertion_point_to_start(pkg.ir.Block()) or b.create_program_id(3)
    # enum values follow Enums.td
    assert int(pkg.ir.MatmulImplWay.MMA_M16N8K16_F8) == 4 and int(pkg.ir.RoundingMode.RN) == 1
    assert int(pkg.ir.PaddingOption.NINF) == 3 and int(pkg.ir.EvictPriority.NO_ALLOCATE) == 4


def test_downcast_needs_rounding_mode(pkg):
    ir = pkg.ir
    b = ir.Builder()
    blk = ir.Block([ir.TensorType((1, 8), ir.Type("f32"))])
    b.set_insertion_point_to_start(blk)
    with pytest.raises(ValueError, match="rounding mode must be set"):
        b.create_fptofp(ir.TensorType((1, 8), ir.Type("bf16")), blk.args[0], None)
    b.create_fptofp(ir.TensorType((1, 8), ir.Type("bf16")), blk.args[0], ir.RoundingMode.RZ)


def test_lifting_elementwise_to_one_call(pkg):
    mod, fn = build_affine_gelu(pkg)
    n = 1024 * 6
    x, y = torch.zeros(n, dtype=torch.bfloat16), torch.zeros(n, dtype=torch.bfloat16)
    h = FakeHandle()
    pkg.executor.launch(fn, (5, 1, 1), [x, y, n], h, module=mod)   # 5 programs of 4 warps
    assert len(h.log) == 1 and h.log[0][0] == "elementwise"
    _, insts, tin, tout = h.log[0]
    assert (tout.size0, tout.size1, tout.offset_elems) == (1, 5 * 1024, 0)
    assert (tin[0].size0, tin[0].size1) == (1, 5 * 1024) and tin[0].ptr == x.data_ptr()
    ops = [t[0] for t in insts]
    A = pkg.abi
    assert ops.count(A.OP_EXP) == 1 and ops.count(A.OP_DIV) == 1 and ops[-1] == A.OP_STORE
    assert max(t[2] for t in insts) < A.MAX_REGS
    # a grid that overshoots the tensor is clipped to it (stores are predicated)
    h2 = FakeHandle()
    pkg.executor.launch(fn, (8, 1, 1), [x, y, n], h2, module=mod)
    assert h2.log[0][3].size1 == n


def test_cache_hints_reach_the_descriptors(pkg):
    """CacheModifier / EvictPriority / volatile given to create_ld_global and
    create_st_global (ir.cc:1035-1049) arrive in kapyb_tensor2d.cache."""
    ir = pkg.ir
    b = ir.Builder(ir.MLIRContext())
    mod = b.create_module()
    mod.set_attr("kapy.num_warps", 1)
    ptr, i32 = b.get_pointer_type(1), b.get_int32_type()
    fn = b.get_or_create_function(mod, "k", b.get_function_type([ptr, ptr, i32], []), "public", False)
    mod.push_back(fn)
    b.set_insertion_point_to_start(fn.add_entry_block())
    x, y, n = fn.get_argument(0), fn.get_argument(1), fn.get_argument(2)
    f32 = b.get_float32_type()
    c0, c1, c256 = b.create_constant_int32(0), b.create_constant_int32(1), b.create_constant_int32(256)
    gx, gy = b.create_mk_global(x, c0, c1, n, n, c1, f32), b.create_mk_global(y, c0, c1, n, n, c1, f32)
    lo = b.create_muli(b.create_program_id(0), c256)
    hi = b.create_addi(lo, c256)
    vx, vy = b.create_sv_global(gx, c0, c1, lo, hi, [1, 256]), b.create_sv_global(gy, c0, c1, lo, hi, [1, 256])
    t = b.create_ld_global(vx, ir.PaddingOption.ZERO, ir.CacheModifier.NONE, ir.EvictPriority.EVICT_FIRST, False)
    b.create_st_global(b.create_absf(t), vy, ir.CacheModifier.CS, ir.EvictPriority.EVICT_NORMAL, False)
    b.create_return([])
    fn.finalize()
    h = FakeHandle()
    xs, ys = torch.zeros(1024), torch.zeros(1024)
    pkg.executor.launch(fn, (4, 1, 1), [xs, ys, 1024], h, module=mod)
    _, insts, tin, tout = h.log[0]
    A = pkg.abi
    assert tin[0].cache == A.cache_hints(A.CACHE_NONE, A.EVICT_FIRST, False)
    assert tout.cache == A.cache_hints(A.CACHE_CS, A.EVICT_NORMAL, False)


def test_lifting_rejects_what_it_cannot_lift(pkg):
    ir = pkg.ir
    b = ir.Builder()
    mod = b.create_module()
    ptr = b.get_pointer_type(1)
    fn = b.get_or_create_function(mod, "k", b.get_function_type([ptr, ptr], []), "public", False)
    b.set_insertion_point_to_start(fn.add_entry_block())
    c0, c1, c64 = (b.create_constant_int32(v) for v in (0, 1, 64))
    f16 = b.get_float16_type()
    g = b.create_mk_global(fn.get_argument(0), c0, c1, c64, c64, c1, f16)
    go = b.create_mk_global(fn.get_argument(1), c0, c1, c64, c64, c1, f16)
    pid = b.create_program_id(0)
    # tiles 32 wide but programs 48 apart: the grid leaves gaps
    lo = b.create_muli(pid, b.create_constant_int32(48))
    hi = b.create_addi(lo, b.create_constant_int32(32))
    v = b.create_ld_global(b.create_sv_global(g, c0, c1, lo, hi, [1, 32]))
    b.create_st_global(v, b.create_sv_global(go, c0, c1, lo, hi, [1, 32]))
    b.create_return([])
    t = torch.zeros(64, dtype=torch.float16)
    with pytest.raises(pkg.executor.Unsupported, match="contiguous"):
        pkg.executor.launch(fn, (2, 1, 1), [t, t], FakeHandle(), num_warps=1)


@pytest.mark.gpu
@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
def test_builder_gelu_runs_on_gpu(handle, ko, pkg, dt):
    mod, fn = build_affine_gelu(pkg, "bf16" if dt == torch.bfloat16 else "f16")
    n = 1024 * 40
    x = normal((n,), 1003, dtype=dt)
    xd, yd = x.cuda(), torch.zeros(n, dtype=dt, device="cuda")
    ran = pkg.executor.launch(fn, (40, 1, 1), [xd, yd, n], handle, module=mod)
    handle.check()
    assert ran == ["elt_affine_gelu"]            # the recorded graph hit the fused kernel
    code = pkg.runtime.dtype_code(dt)
    want = ko.eltwise(pkg.programs.affine_gelu_tanh(code, 0.5, 0.1), [bits(x).reshape(1, -1)],
                      [code], (1, n), code)
    assert ko.ulp_diff(bits(yd.cpu()).reshape(1, -1), want).max() <= 2
