"""In-memory kapy IR and a `Builder` with the method names and arities of the
reference's ``ir.Builder`` (python/src/ir.cc:480-1181) for the ops on the
matmul / elementwise / reduce path.

The reference builder emits MLIR that a pass pipeline lowers to PTX text; this
one records the same ops in a small Python IR which ``executor.launch`` lifts
to whole-problem calls of the C ABI.  Op names are the MLIR op names
(``kapy.ld_global``, ``arith.addf``, ``scf.for`` ...), so IR built here and IR
read from ``.mlir`` text (``mlir_text.parse_mlir_module``) look the same to the
executor.  ``create_*`` methods that exist in the reference but are not on the
path raise ``NotImplementedError`` naming themselves.
"""
from __future__ import annotations

import enum
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence


# ------------------------------------------------------------------ enums
# Numeric values follow include/kapy/Dialect/Kapy/IR/Enums.td:42-109.

class MemorySpace(enum.IntEnum):
    GLOBAL_MEMORY = 0
    SHARED_MEMORY = 1
    REGISTER_FILE = 2


class PaddingOption(enum.IntEnum):
    ZERO = 0
    QNAN = 1
    PINF = 2
    NINF = 3


class CacheModifier(enum.IntEnum):
    NONE = 0
    CA = 1
    CG = 2
    CS = 3
    WB = 4
    WT = 5
    LU = 6
    CV = 7


class EvictPriority(enum.IntEnum):
    EVICT_NORMAL = 0
    EVICT_FIRST = 1
    EVICT_LAST = 2
    EVICT_UNCHANGED = 3
    NO_ALLOCATE = 4


class MatmulImplWay(enum.IntEnum):
    MMA_M16N8K8_F16 = 1
    MMA_M16N8K16_F16 = 2
    MMA_M16N8K8_TF32 = 3
    MMA_M16N8K16_F8 = 4


class RoundingMode(enum.IntEnum):
    RZ = 0
    RN = 1


# ------------------------------------------------------------------ types

@dataclass(frozen=True)
class Type:
    kind: str  # 'i1','i8','i16','i32','i64','f16','bf16','f32','f64','f8e4m3','f8e5m2','ptr','none'

    def is_int(self):
        return self.kind in ("i1", "i8", "i16", "i32", "i64")

    def is_float8e4m3(self):
        return self.kind == "f8e4m3"

    def is_float8e5m2(self):
        return self.kind == "f8e5m2"

    def is_bfloat16(self):
        return self.kind == "bf16"

    def is_float16(self):
        return self.kind == "f16"

    def is_float32(self):
        return self.kind == "f32"

    def is_float64(self):
        return self.kind == "f64"

    def is_float(self):
        return self.kind in ("f16", "bf16", "f32", "f64", "f8e4m3", "f8e5m2")

    @property
    def bits(self):
        return {"i1": 1, "i8": 8, "i16": 16, "i32": 32, "i64": 64, "f16": 16, "bf16": 16,
                "f32": 32, "f64": 64, "f8e4m3": 8, "f8e5m2": 8, "ptr": 64}.get(self.kind, 0)

    def __str__(self):
        return "!kapy.ptr<1>" if self.kind == "ptr" else self.kind


@dataclass(frozen=True)
class TensorType:
    shape: tuple            # ints; -1 = dynamic ('?')
    element: Type
    memory: MemorySpace = MemorySpace.REGISTER_FILE

    def __str__(self):
        dims = "x".join("?" if d < 0 else str(d) for d in self.shape)
        enc = {0: "#global", 1: "#shared", 2: "#values"}[int(self.memory)]
        return f"tensor<{dims}x{self.element}, {enc}>"


@dataclass(frozen=True)
class FunctionType:
    inputs: tuple
    results: tuple

    def get_param_types(self):
        return list(self.inputs)


def element_type(t):
    return t.element if isinstance(t, TensorType) else t


# ------------------------------------------------------------------ IR core

class Value:
    def __init__(self, type_, op=None, index=0, name=None):
        self.type = type_
        self.op = op          # defining Operation (None for block arguments)
        self.index = index
        self.name = name
        self.block_arg_of = None
        self.attrs: Dict[str, object] = {}

    def get_type(self):
        return self.type

    def set_attr(self, name, value):
        self.attrs[name] = value

    def __repr__(self):
        return f"<Value {self.name or '?'} : {self.type}>"


class Block:
    def __init__(self, arg_types: Sequence = ()):
        self.args: List[Value] = []
        self.ops: List["Operation"] = []
        self.parent_op: Optional["Operation"] = None
        for t in arg_types:
            self.add_argument(t)

    def add_argument(self, type_):
        v = Value(type_, None, len(self.args))
        v.block_arg_of = self
        self.args.append(v)
        return v

    def get_argument(self, i):
        return self.args[i]

    def get_num_arguments(self):
        return len(self.args)

    def has_terminator(self):
        return bool(self.ops) and self.ops[-1].name in ("kapy.return", "scf.yield", "scf.condition")

    def has_return(self):
        return bool(self.ops) and self.ops[-1].name == "kapy.return"


class Region:
    def __init__(self):
        self.blocks: List[Block] = []

    def size(self):
        return len(self.blocks)

    def empty(self):
        return not self.blocks


class Operation:
    def __init__(self, name, operands=(), result_types=(), attrs=None, n_regions=0):
        self.name = name
        self.operands: List[Value] = list(operands)
        self.results: List[Value] = [Value(t, self, i) for i, t in enumerate(result_types)]
        self.attrs: Dict[str, object] = dict(attrs or {})
        self.regions: List[Region] = [Region() for _ in range(n_regions)]
        self.parent_block: Optional[Block] = None

    def get_num_operands(self):
        return len(self.operands)

    def get_operand(self, i):
        return self.operands[i]

    def get_num_results(self):
        return len(self.results)

    def get_result(self, i):
        if i >= len(self.results):
            raise IndexError("op result index out of range")   # py::index_error, ir.cc:313
        return self.results[i]

    def get_num_regions(self):
        return len(self.regions)

    def get_region(self, i):
        if i >= len(self.regions):
            raise IndexError("op region index out of range")
        return self.regions[i]

    def set_attr(self, name, value):
        self.attrs[name] = value

    def get_name(self):
        return self.name

    # scf.for helpers (ir.cc ForOp bindings)
    def get_induction_var(self):
        return self.regions[0].blocks[0].args[0]

    def get_body(self, i=0):
        return self.regions[0].blocks[i]

    def __repr__(self):
        return f"<Op {self.name}>"


class FuncOp(Operation):
    def __init__(self, name, ftype: FunctionType, visibility="public", noinline=False):
        super().__init__("kapy.func", (), (), {"sym_name": name, "sym_visibility": visibility,
                                               "noinline": noinline}, n_regions=1)
        self.function_type = ftype
        self.arg_attrs: List[Dict[str, int]] = [dict() for _ in ftype.inputs]

    @property
    def sym_name(self):
        return self.attrs["sym_name"]

    def add_entry_block(self):
        blk = Block(self.function_type.inputs)
        blk.parent_op = self
        self.regions[0].blocks.append(blk)
        return blk

    def get_argument(self, index):
        if index >= len(self.function_type.inputs):
            raise IndexError("function argument index out of range")   # ir.cc:439-441
        return self.regions[0].blocks[0].args[index]

    def set_arg_attr(self, index, name, value):
        self.arg_attrs[index][name] = int(value)

    def finalize(self):
        """Drops ops after the first return of each block (ir.cc:452-474)."""
        for blk in self.regions[0].blocks:
            for i, op in enumerate(blk.ops):
                if op.name == "kapy.return":
                    del blk.ops[i + 1:]
                    break

    def set_type(self, ftype):
        self.function_type = ftype


class ModuleOp(Operation):
    def __init__(self):
        super().__init__("builtin.module", (), (), {}, n_regions=1)
        self.functions: Dict[str, FuncOp] = {}

    def push_back(self, func: FuncOp):
        self.functions[func.sym_name] = func

    def has_function(self, name):
        return name in self.functions

    def get_function(self, name):
        return self.functions.get(name)

    def get_int_attr(self, name):
        v = self.attrs.get(name)
        return int(v) if v is not None else None

    def walk(self, callback):
        def rec(op):
            for r in op.regions:
                for b in r.blocks:
                    for o in b.ops:
                        rec(o)
            callback(op)
        for f in self.functions.values():
            rec(f)


class MLIRContext:
    """Stands in for the reference's context object (ir.cc:157-159)."""


def load_dialects(context):   # ir.cc:161-170
    return None


# ------------------------------------------------------------------ builder

_FLOAT_BIN = {"create_mulf": "arith.mulf", "create_divf": "arith.divf", "create_addf": "arith.addf",
              "create_subf": "arith.subf", "create_remf": "arith.remf",
              "create_minimumf": "arith.minimumf", "create_minnumf": "arith.minnumf",
              "create_maximumf": "arith.maximumf", "create_maxnumf": "arith.maxnumf"}
_INT_BIN = {"create_muli": "arith.muli", "create_divsi": "arith.divsi", "create_divui": "arith.divui",
            "create_remsi": "arith.remsi", "create_remui": "arith.remui", "create_addi": "arith.addi",
            "create_subi": "arith.subi", "create_shli": "arith.shli", "create_shrui": "arith.shrui",
            "create_shrsi": "arith.shrsi", "create_minsi": "arith.minsi", "create_minui": "arith.minui",
            "create_maxsi": "arith.maxsi", "create_maxui": "arith.maxui", "create_andi": "arith.andi",
            "create_ori": "arith.ori", "create_xori": "arith.xori"}
_UNARY_MATH = {"create_floor": "math.floor", "create_ceil": "math.ceil", "create_exp": "math.exp",
               "create_exp2": "math.exp2", "create_cos": "math.cos", "create_sin": "math.sin",
               "create_log": "math.log", "create_log2": "math.log2", "create_erf": "math.erf",
               "create_sqrt": "math.sqrt", "create_rsqrt": "math.rsqrt", "create_absf": "math.absf",
               "create_absi": "math.absi"}
_CMPI = ["sle", "slt", "sge", "sgt", "ule", "ult", "uge", "ugt", "eq", "ne"]
_CMPF = ["olt", "ogt", "ole", "oge", "oeq", "one", "ult", "ugt", "ule", "uge", "ueq", "une"]


class Builder:
    """Mirror of ``ir.Builder`` (python/src/ir.cc:480-1181)."""

    def __init__(self, context: Optional[MLIRContext] = None):
        self.context = context
        self._block: Optional[Block] = None
        self._pos: Optional[int] = None   # insertion index inside _block (None = end)
        self._loc = None

    # -- plumbing ---------------------------------------------------------
    def _insert(self, op: Operation) -> Operation:
        if self._block is None:
            raise RuntimeError("no insertion point set")
        op.parent_block = self._block
        if self._pos is None:
            self._block.ops.append(op)
        else:
            self._block.ops.insert(self._pos, op)
            self._pos += 1
        return op

    def _op(self, name, operands, result_types, attrs=None, n_regions=0):
        return self._insert(Operation(name, operands, result_types, attrs, n_regions))

    def _val(self, name, operands, result_type, attrs=None):
        return self._op(name, operands, [result_type], attrs).results[0]

    def create_module(self):
        return ModuleOp()

    def set_insertion_point_to_start(self, block):
        self._block, self._pos = block, 0

    def set_insertion_point_to_end(self, block):
        self._block, self._pos = block, None

    def set_insertion_point_after(self, op):
        self._block = op.parent_block
        self._pos = self._block.ops.index(op) + 1

    def get_insertion_block(self):
        return self._block

    def save_insertion_point(self):
        return (self._block, self._pos)

    def restore_insertion_point(self, ip):
        self._block, self._pos = ip

    def get_bool_attr(self, value):
        return bool(value)

    def get_int64_attr(self, value):
        return int(value)

    def set_loc(self, *args):
        self._loc = args

    def get_loc(self):
        return self._loc

    # -- types ------------------------------------------------------------
    def get_void_type(self):
        return Type("none")

    def get_int1_type(self):
        return Type("i1")

    def get_int8_type(self):
        return Type("i8")

    def get_int16_type(self):
        return Type("i16")

    def get_int32_type(self):
        return Type("i32")

    def get_int64_type(self):
        return Type("i64")

    def get_float8e4m3_type(self):
        return Type("f8e4m3")

    def get_float8e5m2_type(self):
        return Type("f8e5m2")

    def get_bfloat16_type(self):
        return Type("bf16")

    def get_float16_type(self):
        return Type("f16")

    def get_float32_type(self):
        return Type("f32")

    def get_pointer_type(self, space=1):
        return Type("ptr")

    def get_tensor_type(self, shape, element_type, memory):
        return TensorType(tuple(shape), element_type, MemorySpace(memory))

    def get_function_type(self, inputs, results):
        return FunctionType(tuple(inputs), tuple(results))

    # -- constants --------------------------------------------------------
    def _const(self, value, type_):
        return self._val("arith.constant", [], type_, {"value": value})

    def create_constant_int1(self, v):
        return self._const(bool(v), Type("i1"))

    def create_constant_int8(self, v):
        return self._const(int(v), Type("i8"))

    def create_constant_int16(self, v):
        return self._const(int(v), Type("i16"))

    def create_constant_int32(self, v):
        return self._const(int(v), Type("i32"))

    def create_constant_int64(self, v):
        return self._const(int(v), Type("i64"))

    def create_constant_bfloat16(self, v):
        return self._const(float(v), Type("bf16"))

    def create_constant_float16(self, v):
        return self._const(float(v), Type("f16"))

    def create_constant_float32(self, v):
        return self._const(float(v), Type("f32"))

    def create_constant_float64(self, v):
        return self._const(float(v), Type("f64"))

    def create_constant_zero(self, type_):
        if isinstance(type_, Type) and (type_.is_float() or type_.is_int()):
            return self._const(0.0 if type_.is_float() else 0, type_)
        raise RuntimeError("not implemented")                      # ir.cc:588

    def create_constant_all_ones(self, type_):
        if isinstance(type_, Type) and type_.is_int():
            return self._const((1 << type_.bits) - 1, type_)
        raise RuntimeError("not implemented")

    # -- functions / control flow -----------------------------------------
    def get_or_create_function(self, module, name, type_, visibility, noinline):
        if module.has_function(name):
            return module.get_function(name)
        if not isinstance(type_, FunctionType):
            raise ValueError("invalid function type")               # std::invalid_argument, ir.cc:677
        f = FuncOp(name, type_, visibility, noinline)
        return f

    def create_return(self, operands):
        return self._op("kapy.return", operands, [])

    def create_call(self, func, operands):
        return self._op("kapy.call", operands, list(func.function_type.results),
                        {"callee": func.sym_name})

    def create_for(self, lb, ub, step, operands):
        op = self._op("scf.for", [lb, ub, step, *operands], [o.type for o in operands],
                      n_regions=1)
        body = Block([lb.type, *[o.type for o in operands]])
        body.parent_op = op
        op.regions[0].blocks.append(body)
        return op

    def create_yield(self, operands):
        return self._op("scf.yield", operands, [])

    def create_if(self, result_types, condition, with_else):
        op = self._op("scf.if", [condition], list(result_types), n_regions=2)
        for r in op.regions[: 2 if with_else else 1]:
            b = Block()
            b.parent_op = op
            r.blocks.append(b)
        return op

    def create_while(self, result_types, operands):
        raise NotImplementedError("create_while (scf.while) is not on the matmul/elementwise path")

    def create_condition(self, condition, operands):
        raise NotImplementedError("create_condition (scf.condition) is not on the path")

    # -- casts --------------------------------------------------------------
    def _like(self, source, elem):
        t = source.type
        return TensorType(t.shape, elem, t.memory) if isinstance(t, TensorType) else elem

    def create_fptofp(self, result_type, source, rounding_mode=None):
        attrs = {} if rounding_mode is None else {"rounding_mode": RoundingMode(rounding_mode)}
        src_bits, dst_bits = element_type(source.type).bits, element_type(result_type).bits
        if dst_bits < src_bits and rounding_mode is None:
            # FPToFPOp::verify, Kapy.cpp:272-287
            raise ValueError("rounding mode must be set for down cast")
        return self._val("kapy.fptofp", [source], result_type, attrs)

    def create_bitcast(self, result_type, source):
        return self._val("arith.bitcast", [source], result_type)

    def create_sitofp(self, result_type, source):
        return self._val("arith.sitofp", [source], result_type)

    def create_fptosi(self, result_type, source):
        return self._val("arith.fptosi", [source], result_type)

    def create_extf(self, result_type, source):
        return self._val("arith.extf", [source], result_type)

    def create_truncf(self, result_type, source):
        return self._val("arith.truncf", [source], result_type)

    def create_intcast(self, result_type, source, is_signed):
        ob, nb = element_type(source.type).bits, element_type(result_type).bits
        name = ("arith.bitcast" if ob == nb else "arith.trunci" if ob > nb
                else "arith.extsi" if is_signed else "arith.extui")
        return self._val(name, [source], result_type)

    # -- arithmetic ---------------------------------------------------------
    def create_fma(self, lhs, rhs, acc):
        return self._val("math.fma", [lhs, rhs, acc], lhs.type)

    def create_clampf(self, source, low, high, propagate_nan):
        return self._val("kapy.clampf", [source, low, high], source.type,
                         {"propagate_nan": bool(propagate_nan)})

    def create_select(self, condition, true_value, false_value):
        return self._val("arith.select", [condition, true_value, false_value], true_value.type)

    # -- memory -------------------------------------------------------------
    def create_mk_global(self, global_address, dynamic_offset, size0, size1, stride0, stride1,
                         element_type_):
        rt = TensorType((-1, -1), element_type_, MemorySpace.GLOBAL_MEMORY)
        return self._val("kapy.mk_global",
                         [global_address, dynamic_offset, size0, size1, stride0, stride1], rt)

    def create_sv_global(self, source, start0, end0, start1, end1, shape):
        rt = TensorType(tuple(shape), source.type.element, MemorySpace.GLOBAL_MEMORY)
        return self._val("kapy.sv_global", [source, start0, end0, start1, end1], rt)

    def create_ld_global(self, source, padding_option=PaddingOption.ZERO,
                         cache_modifier=CacheModifier.NONE,
                         evict_priority=EvictPriority.EVICT_NORMAL, is_volatile=False):
        rt = TensorType(source.type.shape, source.type.element, MemorySpace.REGISTER_FILE)
        return self._val("kapy.ld_global", [source], rt,
                         {"padding_option": PaddingOption(padding_option),
                          "cache_modifier": CacheModifier(cache_modifier),
                          "evict_priority": EvictPriority(evict_priority),
                          "is_volatile": bool(is_volatile)})

    def create_st_global(self, source, target, cache_modifier=CacheModifier.NONE,
                         evict_priority=EvictPriority.EVICT_NORMAL, is_volatile=False):
        self._op("kapy.st_global", [source, target], [],
                 {"cache_modifier": CacheModifier(cache_modifier),
                  "evict_priority": EvictPriority(evict_priority), "is_volatile": bool(is_volatile)})

    def create_mk_shared(self, shape, element_type_, row_major):
        rt = TensorType(tuple(shape), element_type_, MemorySpace.SHARED_MEMORY)
        return self._val("kapy.mk_shared", [], rt, {"kapy.row_major": bool(row_major)})

    def create_sv_shared(self, source, start0, end0, start1, end1, shape):
        rt = TensorType(tuple(shape), source.type.element, MemorySpace.SHARED_MEMORY)
        return self._val("kapy.sv_shared", [source, start0, end0, start1, end1], rt)

    def create_splat(self, source, shape):
        return self._val("kapy.splat", [source], TensorType(tuple(shape), source.type))

    def create_broadcast(self, source, shape):
        if not isinstance(source.type, TensorType):
            raise ValueError("source must be a tensor")              # ir.cc:1085
        rt = TensorType(tuple(shape), source.type.element, source.type.memory)
        return self._val("kapy.broadcast", [source], rt)

    def create_transpose(self, source):
        s = source.type.shape
        return self._val("kapy.transpose", [source],
                         TensorType((s[1], s[0]), source.type.element, source.type.memory))

    def create_arange(self, axis, start, end):
        if axis > 1:
            raise IndexError("program axis must be 0, 1")            # ir.cc:734
        shape = (end - start, 1) if axis == 0 else (1, end - start)
        return self._val("kapy.arange", [], TensorType(shape, Type("i32")),
                         {"axis": axis, "start": start, "end": end})

    def create_program_id(self, axis):
        if axis > 2:
            raise IndexError("program axis must be 0, 1, 2")         # ir.cc:1094
        return self._val("kapy.program_id", [], Type("i32"), {"axis": int(axis)})

    def create_warp_id(self):
        return self._val("kapy.warp_id", [], Type("i32"))

    def create_lane_id(self):
        return self._val("kapy.lane_id", [], Type("i32"))

    def create_matmul(self, lhs, rhs, acc, impl_way):
        return self._val("kapy.matmul", [lhs, rhs, acc], acc.type,
                         {"matmul_impl_way": MatmulImplWay(impl_way)})

    def create_reduce(self, source, axis):
        s = list(source.type.shape)
        s[axis] = 1
        op = self._op("kapy.reduce", [source],
                      [TensorType(tuple(s), source.type.element, source.type.memory)],
                      {"axis": int(axis)}, n_regions=1)
        e = source.type.element
        body = Block([e, e])
        body.parent_op = op
        op.regions[0].blocks.append(body)
        return op

    def create_elementwise_extern_lib(self, result_type, operands, lib_name, lib_path, sym_name,
                                      pure):
        return self._val("kapy.elementwise_extern_lib", list(operands), result_type,
                         {"lib_name": lib_name, "lib_path": lib_path, "sym_name": sym_name,
                          "pure": bool(pure)})

    def create_elementwise_inline_asm(self, *args):
        raise NotImplementedError("create_elementwise_inline_asm: inline PTX cannot be lifted to "
                                  "the pre-compiled kernels")

    def __getattr__(self, name):
        # Families of same-shaped creators.
        if name in _FLOAT_BIN or name in _INT_BIN:
            opname = _FLOAT_BIN.get(name) or _INT_BIN[name]
            return lambda lhs, rhs: self._val(opname, [lhs, rhs], lhs.type)
        if name in _UNARY_MATH:
            opname = _UNARY_MATH[name]
            return lambda source: self._val(opname, [source], source.type)
        if name.startswith("create_cmpi_") and name[12:] in _CMPI:
            pred = name[12:]
            return lambda lhs, rhs: self._val("arith.cmpi", [lhs, rhs],
                                              self._like(lhs, Type("i1")), {"predicate": pred})
        if name.startswith("create_cmpf_") and name[12:] in _CMPF:
            pred = name[12:]
            return lambda lhs, rhs: self._val("arith.cmpf", [lhs, rhs],
                                              self._like(lhs, Type("i1")), {"predicate": pred})
        if name.startswith("create_") or name.startswith("get_"):
            raise NotImplementedError(f"Builder.{name} exists in the reference but is not on the "
                                      "matmul / elementwise / reduce path")
        raise AttributeError(name)


def parse_mlir_module(file_name, context=None):
    """ir.parse_mlir_module (ir.cc:426-434) for the textual kapy IR."""
    from .mlir_text import parse_file
    try:
        return parse_file(file_name)
    except (OSError, SyntaxError) as ex:
        raise RuntimeError("parse mlir module file failed.") from ex
