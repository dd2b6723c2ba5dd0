"""Runs a kapy kernel (built with ``ir.Builder`` or read from text) on the B200
backend by lifting it from the reference's per-warp view to whole-problem
calls of the C ABI.

A kapy kernel describes what ONE warp of ONE program does: it slices fixed-size
tiles out of global tensors with ``kapy.sv_global`` at offsets that are affine
in ``program_id`` / ``warp_id``, computes on register tensors and stores a tile
back (elementwise_add.mlir:9-25, reduce_sum.mlir:10-25, matmul.mlir:1-134).
The reference compiles that text to PTX and leaves launching to the caller.
Here the launch is evaluated symbolically instead: the program/warp ids stay
symbols, the union of the tiles the grid touches becomes a region of the
tensors, and the computation on that region is handed to
``kapyb_elementwise`` / ``kapyb_reduce`` / ``kapyb_matmul`` in one call.

What is recognised:
  * straight-line elementwise graphs whose loads and store use the same tile
    index (any op ``kapyb_inst`` can express, broadcast operands, padding);
  * ``kapy.reduce`` with a single-op lambda over a tile spanning the reduced
    axis, optionally fed by an elementwise graph;
  * matmul kernels: every ``kapy.matmul`` in the function must draw its lhs from
    one global tensor and its rhs from another -- directly (``ld_global``) or
    through shared memory (``cp_async_global_to_shared`` + ``ld_matrix``) -- and
    the stored tile must be the accumulator chain, optionally followed by a
    scale, a broadcast bias add and a downcast.  The software pipeline around
    the matmuls (stages, waits, buffer selects) is the idiom the tcgen05 kernel
    replaces, so it is not executed op by op.
Anything else raises ``Unsupported``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

from . import _abi as abi
from . import ir


class Unsupported(NotImplementedError):
    pass


_DT = {"f16": abi.F16, "bf16": abi.BF16, "f32": abi.F32, "f8e4m3": abi.F8E4M3,
       "f8e5m2": abi.F8E5M2,  # the f8 types: matmul operands only (the library checks)
       "i1": abi.I1}          # conditions of arith.select inside an elementwise graph


_ESZ = {abi.F16: 2, abi.BF16: 2, abi.F32: 4, abi.F8E4M3: 1, abi.F8E5M2: 1}


def _dtype(t) -> int:
    k = ir.element_type(t).kind
    if k not in _DT:
        raise Unsupported(f"element type {k} is not supported by the backend")
    return _DT[k]


# ------------------------------------------------------------ affine scalars

class Affine:
    """const + sum(coeff * symbol); symbols are program/warp ids."""

    def __init__(self, const=0, terms=None):
        self.const = int(const)
        self.terms: Dict[str, int] = {k: int(v) for k, v in (terms or {}).items() if v}

    def is_const(self):
        return not self.terms

    def __add__(self, o):
        t = dict(self.terms)
        for k, v in o.terms.items():
            t[k] = t.get(k, 0) + v
        return Affine(self.const + o.const, t)

    def __sub__(self, o):
        return self + o.scale(-1)

    def scale(self, c):
        return Affine(self.const * c, {k: v * c for k, v in self.terms.items()})

    def same_terms(self, o):
        return self.terms == o.terms

    def __eq__(self, o):
        return isinstance(o, Affine) and self.const == o.const and self.terms == o.terms

    def __repr__(self):
        return " + ".join([str(self.const)] + [f"{v}*{k}" for k, v in self.terms.items()])


@dataclass
class GlobalRoot:
    arg: int              # index of the pointer argument
    offset: int           # dynamic_offset, elements
    size0: int
    size1: int
    stride0: int
    stride1: int
    dtype: int


@dataclass
class GlobalView:
    root: GlobalRoot
    start0: Affine
    end0: Affine
    start1: Affine
    end1: Affine
    shape: Tuple[int, int]


@dataclass
class Expr:
    kind: str                    # load | const | op | reduce | matmul | opaque
    dtype: int = abi.F32
    shape: Tuple[int, int] = (1, 1)
    name: str = ""
    args: tuple = ()
    attrs: dict = None
    view: Optional[GlobalView] = None
    value: float = 0.0


_OPCODES = {
    "arith.addf": abi.OP_ADD, "arith.subf": abi.OP_SUB, "arith.mulf": abi.OP_MUL,
    "arith.divf": abi.OP_DIV, "math.fma": abi.OP_FMA, "arith.maximumf": abi.OP_MAXIMUM,
    "arith.minimumf": abi.OP_MINIMUM, "arith.maxnumf": abi.OP_MAXNUM,
    "arith.minnumf": abi.OP_MINNUM, "kapy.clampf": abi.OP_CLAMP, "math.absf": abi.OP_ABS,
    "arith.negf": abi.OP_NEG, "math.exp": abi.OP_EXP, "math.exp2": abi.OP_EXP2,
    "math.log": abi.OP_LOG, "math.log2": abi.OP_LOG2, "math.sqrt": abi.OP_SQRT,
    "math.rsqrt": abi.OP_RSQRT, "math.erf": abi.OP_ERF, "math.sin": abi.OP_SIN,
    "math.cos": abi.OP_COS, "math.floor": abi.OP_FLOOR, "math.ceil": abi.OP_CEIL,
    "arith.extf": abi.OP_CVT, "arith.truncf": abi.OP_CVT, "kapy.fptofp": abi.OP_CVT,
}
_I1_LOGIC = {"arith.andi": abi.OP_AND, "arith.ori": abi.OP_OR, "arith.xori": abi.OP_XOR}
_COMBINERS = {"arith.addf": abi.RED_ADD, "arith.mulf": abi.RED_MUL,
              "arith.maximumf": abi.RED_MAX, "arith.minimumf": abi.RED_MIN}


def _cache_of(op: ir.Operation) -> int:
    """Cache operator, eviction priority and volatile flag of a ld_global / st_global
    (ir.cc:1035-1049) packed as kapyb_tensor2d.cache wants them."""
    return abi.cache_hints(int(op.attrs.get("cache_modifier", 0)), int(op.attrs.get("evict_priority", 0)),
                           bool(op.attrs.get("is_volatile", False)))


class _Lifter:
    def __init__(self, func: ir.FuncOp, grid, args, num_warps: int):
        self.func = func
        self.args = list(args)
        gx, gy, gz = (list(grid) + [1, 1, 1])[:3]
        self.ranges: Dict[str, int] = {"pid0": gx, "pid1": gy, "pid2": gz, "wid": num_warps}
        self.env: Dict[ir.Value, object] = {}
        self.stores: List[Tuple[Expr, GlobalView]] = []
        self.store_cache: Dict[int, int] = {}      # id(target view) -> cache hints of its st_global
        self.cp_async: List[Tuple[GlobalView, ir.Value]] = []   # (global source, shared target value)
        self.matmuls: List[ir.Operation] = []
        self.loops: List[ir.Operation] = []

    # ---- scalar evaluation -------------------------------------------------
    def scalar(self, v: ir.Value) -> Optional[Affine]:
        r = self.env.get(v)
        return r if isinstance(r, Affine) else None

    def need_const(self, v: ir.Value, what: str) -> int:
        a = self.scalar(v)
        if a is None or not a.is_const():
            raise Unsupported(f"{what} must be known at launch")
        return a.const

    def _int_op(self, op: ir.Operation):
        a, b = self.scalar(op.operands[0]), self.scalar(op.operands[1])
        if a is None or b is None:
            return None
        n = op.name
        if n == "arith.addi":
            return a + b
        if n == "arith.subi":
            return a - b
        if n == "arith.muli":
            if b.is_const():
                return a.scale(b.const)
            if a.is_const():
                return b.scale(a.const)
            return None
        if n in ("arith.divui", "arith.divsi", "arith.remui", "arith.remsi") and b.is_const() and b.const > 0:
            c = b.const
            if a.is_const():
                return Affine(a.const // c if "div" in n else a.const % c)
            # a bare id split by a constant: two fresh symbols (id // c, id % c)
            if a.const == 0 and len(a.terms) == 1 and list(a.terms.values())[0] == 1:
                sym = list(a.terms)[0]
                rng = self.ranges.get(sym)
                if rng is not None and rng % c == 0 or (rng is not None and rng <= c):
                    hi, lo = f"{sym}//{c}", f"{sym}%{c}"
                    self.ranges.setdefault(hi, max(1, -(-rng // c)))
                    self.ranges.setdefault(lo, min(rng, c))
                    return Affine(0, {hi: 1}) if "div" in n else Affine(0, {lo: 1})
        return None

    # ---- walking the function ----------------------------------------------
    def run(self):
        blk = self.func.regions[0].blocks[0]
        if len(self.args) != len(blk.args):
            raise ValueError(f"kernel takes {len(blk.args)} arguments, {len(self.args)} given")
        for v, a in zip(blk.args, self.args):
            if v.type.kind == "ptr":
                self.env[v] = ("ptr", blk.args.index(v))
            elif v.type.is_int():
                self.env[v] = Affine(int(a))
            elif v.type.is_float():
                self.env[v] = Expr("const", _dtype(v.type), (1, 1), value=float(a))
        self.walk(blk)

    def walk(self, blk: ir.Block):
        for op in blk.ops:
            self.visit(op)

    def expr(self, v: ir.Value) -> Expr:
        r = self.env.get(v)
        if isinstance(r, Expr):
            return r
        return Expr("opaque", name=v.op.name if v.op else "block-arg")

    def visit(self, op: ir.Operation):
        n = op.name
        E = self.env
        if n == "arith.constant":
            t = op.results[0].type
            if isinstance(t, ir.TensorType):
                E[op.results[0]] = Expr("const", _dtype(t), t.shape, value=float(op.attrs["value"]))
            elif t.is_float():
                E[op.results[0]] = Expr("const", _dtype(t), (1, 1), value=float(op.attrs["value"]))
            else:
                E[op.results[0]] = Affine(int(op.attrs["value"]))
        elif n == "kapy.program_id":
            E[op.results[0]] = Affine(0, {f"pid{op.attrs['axis']}": 1})
        elif n == "kapy.warp_id":
            E[op.results[0]] = Affine(0, {"wid": 1})
        elif n == "kapy.lane_id":
            raise Unsupported("kernels that depend on lane_id cannot be lifted")
        elif n.startswith("arith.") and n[6:] in ("addi", "subi", "muli", "divui", "divsi", "remui", "remsi"):
            r = self._int_op(op)
            if r is not None:
                E[op.results[0]] = r
        elif n == "kapy.mk_global":
            ptr = E.get(op.operands[0])
            if not (isinstance(ptr, tuple) and ptr[0] == "ptr"):
                raise Unsupported("mk_global address must be a kernel pointer argument")
            vals = [self.need_const(o, "mk_global offset/size/stride") for o in op.operands[1:]]
            E[op.results[0]] = GlobalRoot(ptr[1], vals[0], vals[1], vals[2], vals[3], vals[4],
                                          _dtype(op.results[0].type))
        elif n == "kapy.sv_global":
            src = E.get(op.operands[0])
            bounds = [self.scalar(o) for o in op.operands[1:]]
            shape = op.results[0].type.shape
            if isinstance(src, GlobalRoot):
                if any(b is None for b in bounds):
                    E[op.results[0]] = ("view-unknown", src)
                else:
                    E[op.results[0]] = GlobalView(src, bounds[0], bounds[1], bounds[2], bounds[3], shape)
            elif isinstance(src, GlobalView) and all(b is not None for b in bounds):
                E[op.results[0]] = GlobalView(src.root, src.start0 + bounds[0], src.start0 + bounds[1],
                                              src.start1 + bounds[2], src.start1 + bounds[3], shape)
            elif isinstance(src, tuple) and src[0] == "view-unknown":
                E[op.results[0]] = src
            else:
                raise Unsupported("sv_global of an unknown source")
        elif n == "kapy.ld_global":
            src = E.get(op.operands[0])
            t = op.results[0].type
            if isinstance(src, GlobalView):
                E[op.results[0]] = Expr("load", _dtype(t), t.shape, view=src,
                                        attrs={"padding": int(op.attrs.get("padding_option", 0)),
                                               "cache": _cache_of(op)})
            elif isinstance(src, tuple):
                E[op.results[0]] = Expr("load-unknown", _dtype(t), t.shape, attrs={"root": src[1]})
            else:
                raise Unsupported("ld_global of something that is not a global view")
        elif n == "kapy.st_global":
            tgt = E.get(op.operands[1])
            if not isinstance(tgt, GlobalView):
                raise Unsupported("st_global target must be a sub-view with launch-time bounds")
            self.stores.append((self.expr(op.operands[0]), tgt))
            self.store_cache[id(tgt)] = _cache_of(op)
        elif n in ("kapy.splat", "kapy.broadcast"):
            src = self.expr(op.operands[0])
            t = op.results[0].type
            E[op.results[0]] = Expr("op", _dtype(t), t.shape, name="broadcast", args=(src,))
        elif n in _OPCODES:
            t = op.results[0].type
            attrs = {}
            if n in ("arith.extf", "arith.truncf"):
                attrs["rounding"] = abi.RN
            elif n == "kapy.fptofp":
                attrs["rounding"] = int(op.attrs.get("rounding_mode", ir.RoundingMode.RN))
            elif n == "kapy.clampf":
                attrs["propagate_nan"] = bool(op.attrs.get("propagate_nan", False))
            shape = t.shape if isinstance(t, ir.TensorType) else (1, 1)
            E[op.results[0]] = Expr("op", _dtype(t), shape, name=n,
                                    args=tuple(self.expr(o) for o in op.operands), attrs=attrs)
        elif n == "arith.cmpf" and self._register_tensor(op.results[0].type):
            # a condition over register tensors: part of an elementwise graph
            t = op.results[0].type
            pred = str(op.attrs.get("predicate", "")).lower()
            if pred not in abi.CMP_PREDICATES:
                raise Unsupported(f"cmpf predicate {pred!r} is not one Builder.create_cmpf_* offers")
            E[op.results[0]] = Expr("op", abi.I1, t.shape, name=n,
                                    args=tuple(self.expr(o) for o in op.operands),
                                    attrs={"predicate": abi.CMP_PREDICATES.index(pred)})
        elif n in _I1_LOGIC and self._register_tensor(op.results[0].type) and \
                op.results[0].type.element.kind == "i1":
            t = op.results[0].type
            E[op.results[0]] = Expr("op", abi.I1, t.shape, name=n,
                                    args=tuple(self.expr(o) for o in op.operands), attrs={})
        elif n == "arith.select" and self._register_tensor(op.results[0].type) and \
                op.results[0].type.element.is_float():
            t = op.results[0].type
            E[op.results[0]] = Expr("op", _dtype(t), t.shape, name=n,
                                    args=tuple(self.expr(o) for o in op.operands), attrs={})
        elif n == "kapy.elementwise_extern_lib":
            if op.attrs.get("sym_name") != "__nv_tanhf":
                raise Unsupported(f"extern function {op.attrs.get('sym_name')} is not available")
            t = op.results[0].type
            E[op.results[0]] = Expr("op", _dtype(t), t.shape, name="tanh",
                                    args=tuple(self.expr(o) for o in op.operands), attrs={})
        elif n == "kapy.reduce":
            body = op.regions[0].blocks[0]
            real = [o for o in body.ops if o.name != "kapy.return"]
            if len(real) != 1 or real[0].name not in _COMBINERS or \
                    set(real[0].operands) != set(body.args):
                raise Unsupported("reduce lambda must be a single add/mul/maximum/minimum of its arguments")
            t = op.results[0].type
            E[op.results[0]] = Expr("reduce", _dtype(t), t.shape, args=(self.expr(op.operands[0]),),
                                    attrs={"axis": int(op.attrs["axis"]),
                                           "combiner": _COMBINERS[real[0].name]})
        elif n == "kapy.matmul":
            self.matmuls.append(op)
            t = op.results[0].type
            E[op.results[0]] = Expr("matmul", _dtype(t), t.shape, attrs={"op": op})
        elif n == "kapy.cp_async_global_to_shared":
            src = E.get(op.operands[0])
            root = src.root if isinstance(src, GlobalView) else (src[1] if isinstance(src, tuple) else None)
            if root is None:
                raise Unsupported("cp_async source must be a global view")
            self.cp_async.append((root, op.operands[1]))
        elif n == "scf.for":
            self.loops.append(op)
            body = op.regions[0].blocks[0]
            # induction variable and iter_args stay symbolic; remember the plumbing
            for barg, init in zip(body.args[1:], op.operands[3:]):
                E[barg] = ("iter", init, op)
            self.walk(body)
            yld = body.ops[-1] if body.ops and body.ops[-1].name == "scf.yield" else None
            for i, r in enumerate(op.results):
                E[r] = ("loop-result", op, i, yld.operands[i] if yld else None)
        elif n in ("kapy.mk_shared", "kapy.sv_shared", "kapy.ld_matrix", "arith.select", "arith.cmpi",
                   "kapy.cp_async_wait_group", "kapy.return", "scf.yield", "arith.cmpf"):
            pass   # plumbing of the software pipeline; followed structurally by trace_root()
        else:
            raise Unsupported(f"op {n} cannot be lifted")

    @staticmethod
    def _register_tensor(t) -> bool:
        return isinstance(t, ir.TensorType) and t.memory == ir.MemorySpace.REGISTER_FILE

    # ---- matmul idiom ------------------------------------------------------
    def trace_roots(self, v: ir.Value, seen=None) -> set:
        """Global tensors a register/shared value is (transitively) filled from."""
        seen = seen if seen is not None else set()
        if v in seen:
            return set()
        seen.add(v)
        r = self.env.get(v)
        if isinstance(r, Expr) and r.kind == "load":
            return {id(r.view.root)}
        if isinstance(r, Expr) and r.kind == "load-unknown":
            return {id(r.attrs["root"])}
        if isinstance(r, tuple) and r[0] == "iter":
            out = self.trace_roots(r[1], seen)
            loop = r[2]
            body = loop.regions[0].blocks[0]
            idx = body.args.index(v) - 1
            yld = body.ops[-1]
            if yld.name == "scf.yield":
                out |= self.trace_roots(yld.operands[idx], seen)
            return out
        if isinstance(r, tuple) and r[0] == "loop-result":
            out = set()
            if r[3] is not None:
                out |= self.trace_roots(r[3], seen)
            out |= self.trace_roots(r[1].operands[3 + r[2]], seen)
            return out
        op = v.op
        if op is None:
            return set()
        if op.name == "kapy.mk_shared":
            out = set()
            for root, target in self.cp_async:
                if self.shared_base(target) is op:
                    out.add(id(root))
            return out
        if op.name in ("kapy.ld_matrix", "kapy.sv_shared", "kapy.transpose"):
            return self.trace_roots(op.operands[0], seen)
        if op.name == "arith.select":
            return self.trace_roots(op.operands[1], seen) | self.trace_roots(op.operands[2], seen)
        return set()

    def shared_base(self, v: ir.Value):
        while v.op is not None and v.op.name in ("kapy.sv_shared",):
            v = v.op.operands[0]
        if v.op is not None and v.op.name == "arith.select":
            return None   # resolved through trace_roots on each branch
        return v.op

    def roots_by_id(self):
        return {id(r): r for r in self.env.values() if isinstance(r, GlobalRoot)}


def _cover(start: Affine, tile: int, ranges: Dict[str, int]) -> Tuple[int, int]:
    """Union over all symbol values of [start, start+tile): must be one interval."""
    terms = sorted(((c, s) for s, c in start.terms.items() if ranges.get(s, 1) > 1))
    for s in start.terms:
        if s not in ranges:
            raise Unsupported(f"tile offset depends on {s}, which has no launch range")
    span = tile
    for c, s in terms:
        if c != span:
            raise Unsupported("tiles of the grid do not cover a contiguous region "
                              f"(step {c} after a span of {span})")
        span *= ranges[s]
    return start.const, start.const + span


class _Program:
    """Turns an expression DAG into kapyb_inst tuples with register reuse."""

    def __init__(self):
        self.insts: List[tuple] = []
        self.inputs: List[Tuple[GlobalView, int, int]] = []   # (view, padding, cache hints)
        self.memo: Dict[int, int] = {}
        self.free = list(range(abi.MAX_REGS - 1, -1, -1))
        self.uses: Dict[int, int] = {}

    def count(self, e: Expr):
        self.uses[id(e)] = self.uses.get(id(e), 0) + 1
        if self.uses[id(e)] == 1:
            for a in e.args:
                self.count(a)

    def release(self, e: Expr):
        self.uses[id(e)] -= 1
        if self.uses[id(e)] == 0 and id(e) in self.memo:
            self.free.append(self.memo[id(e)])

    def alloc(self):
        if not self.free:
            raise Unsupported("elementwise graph needs more than 16 live values")
        return self.free.pop()

    def emit(self, e: Expr) -> int:
        if id(e) in self.memo:
            return self.memo[id(e)]
        if e.kind == "load":
            key = None
            for i, (v, pad, _) in enumerate(self.inputs):
                if v is e.view:
                    key = i
            if key is None:
                if len(self.inputs) >= abi.MAX_INPUTS:
                    raise Unsupported(f"more than {abi.MAX_INPUTS} input tensors")
                self.inputs.append((e.view, e.attrs["padding"], e.attrs.get("cache", 0)))
                key = len(self.inputs) - 1
            r = self.alloc()
            self.insts.append((abi.OP_LOAD, e.dtype, r, -1, -1, -1, 0.0, key))
        elif e.kind == "const":
            r = self.alloc()
            self.insts.append((abi.OP_CONST, e.dtype, r, -1, -1, -1, float(e.value), 0))
        elif e.kind == "op" and e.name == "broadcast":
            r = self.emit(e.args[0])
            self.memo[id(e)] = r
            self.uses[id(e.args[0])] += self.uses.get(id(e), 1) - 1
            return r
        elif e.kind == "op":
            srcs = [self.emit(a) for a in e.args]
            for a in e.args:
                self.release(a)
            r = self.alloc()
            s = srcs + [-1] * (3 - len(srcs))
            if e.name == "tanh":
                code, flags = abi.OP_TANH, 0
            elif e.name == "arith.cmpf":
                code, flags = abi.OP_CMP, int(e.attrs["predicate"])
            elif e.name == "arith.select":
                code, flags = abi.OP_SELECT, 0
            elif e.name in _I1_LOGIC:
                code, flags = _I1_LOGIC[e.name], 0
            else:
                code = _OPCODES[e.name]
                flags = e.attrs.get("rounding", 0) if code == abi.OP_CVT else \
                    int(e.attrs.get("propagate_nan", False)) if code == abi.OP_CLAMP else 0
            self.insts.append((code, e.dtype, r, s[0], s[1], s[2], 0.0, flags))
        else:
            raise Unsupported(f"a {e.kind} value cannot appear inside an elementwise graph")
        self.memo[id(e)] = r
        return r


def _tensor_desc(root: GlobalRoot, tensors, lo0, hi0, lo1, hi1, padding=abi.PAD_ZERO, cache=0):
    t = tensors[root.arg]
    s0 = max(0, min(hi0, root.size0) - lo0)
    s1 = max(0, min(hi1, root.size1) - lo1)
    esz = _ESZ[root.dtype]
    if t.element_size() != esz:
        raise ValueError(f"argument {root.arg} has {t.element_size()}-byte elements but the kernel "
                         f"declares a {esz}-byte element type")
    off = root.offset + lo0 * root.stride0 + lo1 * root.stride1
    return abi.Tensor2d(t.data_ptr(), off, s0, s1, root.stride0, root.stride1, root.dtype, padding,
                        int(cache), 0)


def launch(func, grid: Sequence[int], args: Sequence, handle, num_warps: Optional[int] = None,
           module: Optional[ir.ModuleOp] = None, stream=None) -> List[str]:
    """Executes `func` as if launched on `grid` programs of `num_warps` warps.
    `args`: torch CUDA tensors for pointer parameters, Python numbers for scalars.
    Returns the names of the library kernels that ran."""
    import ctypes as C
    if isinstance(func, ir.ModuleOp):
        module = func
        if len(module.functions) != 1:
            raise ValueError("pass the FuncOp to launch when the module has several functions")
        func = next(iter(module.functions.values()))
    if num_warps is None:
        # getNumWarps falls back to 4 when the module attribute is missing (Kapy.cpp:849-863)
        num_warps = (module.get_int_attr("kapy.num_warps") if module is not None else None) or 4
    L = _Lifter(func, grid, args, num_warps)
    L.run()
    if not L.stores:
        return []
    lib = handle._lib
    ran: List[str] = []
    sp = handle._stream(stream)

    def check(st):
        if st != abi.OK:
            handle._raise(st)

    if L.matmuls:
        ran.append(_launch_matmul(L, handle, sp))
        return ran

    for expr, tgt in L.stores:
        lo0, hi0 = _cover(tgt.start0, tgt.shape[0], L.ranges)
        lo1, hi1 = _cover(tgt.start1, tgt.shape[1], L.ranges)
        if expr.kind == "reduce":
            ran.append(_launch_reduce(L, expr, tgt, (lo0, hi0, lo1, hi1), handle, sp))
            continue
        ran.append(_launch_elementwise(L, expr, tgt, (lo0, hi0, lo1, hi1), handle, sp))
    return ran


def _check_aligned(view: GlobalView, tgt: GlobalView, axis_is_broadcast=(False, False)):
    for ax, (vs, ts) in enumerate(((view.start0, tgt.start0), (view.start1, tgt.start1))):
        if view.shape[ax] == 1 and tgt.shape[ax] != 1:
            if not vs.is_const():
                raise Unsupported("a broadcast operand must not move along its broadcast axis")
            continue
        if not vs.same_terms(ts):
            raise Unsupported("loads and the store of an elementwise kernel must use the same tile index")


def _launch_elementwise(L, expr, tgt, region, handle, sp, out_override=None):
    import ctypes as C
    lo0, hi0, lo1, hi1 = region
    prog = _Program()
    prog.count(expr)
    src = prog.emit(expr)
    out_dtype = expr.dtype
    prog.insts.append((abi.OP_STORE, out_dtype, -1, src, -1, -1, 0.0, 0))
    tin = (abi.Tensor2d * max(1, len(prog.inputs)))()
    for i, (view, pad, cache) in enumerate(prog.inputs):
        _check_aligned(view, tgt)
        b0 = view.shape[0] == 1 and tgt.shape[0] != 1
        b1 = view.shape[1] == 1 and tgt.shape[1] != 1
        v0 = (view.start0.const, view.start0.const + 1) if b0 else \
            (lo0 - tgt.start0.const + view.start0.const, hi0 - tgt.start0.const + view.start0.const)
        v1 = (view.start1.const, view.start1.const + 1) if b1 else \
            (lo1 - tgt.start1.const + view.start1.const, hi1 - tgt.start1.const + view.start1.const)
        tin[i] = _tensor_desc(view.root, L.args, v0[0], v0[1], v1[0], v1[1], pad, cache)
    if out_override is not None:
        tout = out_override
    else:
        if tgt.root.dtype != out_dtype:
            raise ValueError("st_global: source and target element types differ")
        tout = _tensor_desc(tgt.root, L.args, lo0, hi0, lo1, hi1, cache=L.store_cache.get(id(tgt), 0))
    insts = (abi.Inst * len(prog.insts))(*[abi.Inst(*t) for t in prog.insts])
    st = handle._lib.kapyb_elementwise(handle._h, insts, len(prog.insts), tin, len(prog.inputs),
                                       C.byref(tout), sp)
    if st != abi.OK:
        handle._raise(st)
    return handle.last_kernel


def _launch_reduce(L, expr, tgt, region, handle, sp):
    import ctypes as C

    import torch
    lo0, hi0, lo1, hi1 = region
    axis, comb = expr.attrs["axis"], expr.attrs["combiner"]
    src = expr.args[0]
    # the source tile must span the reduced axis from its start
    def src_region(view):
        if axis == 1:
            if not view.start1.is_const() or view.start1.const != 0:
                raise Unsupported("the reduced tile must start at 0 along the reduced axis")
            return (lo0, hi0, 0, view.shape[1])
        if not view.start0.is_const() or view.start0.const != 0:
            raise Unsupported("the reduced tile must start at 0 along the reduced axis")
        return (0, view.shape[0], lo1, hi1)
    keep = None
    if src.kind == "load":
        view = src.view
        other = (view.start0, tgt.start0) if axis == 1 else (view.start1, tgt.start1)
        if not other[0].same_terms(other[1]):
            raise Unsupported("reduce source and target must use the same tile index")
        r = src_region(view)
        root = view.root
        full = root.size1 if axis == 1 else root.size0
        if (r[3] - r[2] if axis == 1 else r[1] - r[0]) < full:
            raise Unsupported("the reduced tile does not span the tensor's reduced axis")
        tsrc = _tensor_desc(root, L.args, r[0], r[1], r[2], r[3])
    else:
        # elementwise producer: materialise it, then reduce
        loads = []
        def collect(e):
            if e.kind == "load":
                loads.append(e)
            for a in e.args:
                collect(a)
        collect(src)
        if not loads:
            raise Unsupported("reduce of a constant")
        r = src_region(loads[0].view)
        rows = max(0, min(r[1], loads[0].view.root.size0) - r[0])
        cols = max(0, min(r[3], loads[0].view.root.size1) - r[2])
        tdt = {abi.F16: torch.float16, abi.BF16: torch.bfloat16, abi.F32: torch.float32}[src.dtype]
        keep = torch.empty((rows, cols), dtype=tdt, device=L.args[loads[0].view.root.arg].device)
        tmp = abi.Tensor2d(keep.data_ptr(), 0, rows, cols, cols, 1, src.dtype, 0)
        fake_tgt = GlobalView(loads[0].view.root, loads[0].view.start0, loads[0].view.end0,
                              loads[0].view.start1, loads[0].view.end1, loads[0].view.shape)
        _launch_elementwise(L, src, fake_tgt, r, handle, sp, out_override=tmp)
        tsrc = tmp
    tdst = _tensor_desc(tgt.root, L.args, lo0, hi0, lo1, hi1)
    # the library infers nothing: shapes must already agree (Kapy.cpp:613-626)
    st = handle._lib.kapyb_reduce(handle._h, C.byref(tsrc), C.byref(tdst), axis, comb, sp)
    if st != abi.OK:
        handle._raise(st)
    if keep is not None:
        handle.check()   # the temporary must outlive the kernels that use it
    return handle.last_kernel


def _launch_matmul(L, handle, sp):
    import ctypes as C
    if len(L.stores) != 1:
        raise Unsupported("a matmul kernel must store exactly one tile")
    expr, tgt = L.stores[0]
    roots = L.roots_by_id()
    lhs_ids, rhs_ids = set(), set()
    for op in L.matmuls:
        lhs_ids |= L.trace_roots(op.operands[0])
        rhs_ids |= L.trace_roots(op.operands[1])
    if len(lhs_ids) != 1 or len(rhs_ids) != 1:
        raise Unsupported("every matmul must read its lhs from one global tensor and its rhs from another")
    A, B = roots[next(iter(lhs_ids))], roots[next(iter(rhs_ids))]
    Cr = tgt.root
    # epilogue between the accumulator chain and the store
    # The fused epilogue computes downcast(act(alpha * acc + bias)): walking back
    # from the store, an activation may only appear before any add / multiply.
    alpha, bias_root, out_dtype, rounding = 1.0, None, expr.dtype, abi.RN
    activation, seen_affine, seen_mul = abi.ACT_NONE, False, False
    e = expr
    while e.kind == "op":
        if e.name in ("arith.truncf", "kapy.fptofp", "arith.extf"):
            rounding = e.attrs.get("rounding", abi.RN)
            e = e.args[0]
        elif e.name in ("arith.maximumf", "arith.maxnumf") and \
                any(_is_splat_const(a) and _splat_value(a) == 0.0 for a in e.args):
            # max(x, 0): relu
            o = [a for a in e.args if not (_is_splat_const(a) and _splat_value(a) == 0.0)]
            if len(o) != 1 or seen_affine or activation != abi.ACT_NONE:
                raise Unsupported("matmul epilogue: relu is recognised once, as the last "
                                  "arithmetic before the store")
            activation = abi.ACT_RELU
            e = o[0]
        elif e.name == "arith.mulf":
            seen_affine = seen_mul = True
            c = [a for a in e.args if _is_splat_const(a)]
            o = [a for a in e.args if not _is_splat_const(a)]
            if len(c) != 1 or len(o) != 1:
                raise Unsupported("matmul epilogue: only a multiply by a constant is recognised")
            alpha *= _splat_value(c[0])
            e = o[0]
        elif e.name == "arith.addf":
            if seen_mul:
                # (acc + bias) * c is not alpha * acc + bias
                raise Unsupported("matmul epilogue: a bias add inside a multiply is not recognised")
            seen_affine = True
            b = [a for a in e.args if _bias_load(a) is not None]
            o = [a for a in e.args if _bias_load(a) is None]
            if len(b) != 1 or len(o) != 1:
                raise Unsupported("matmul epilogue: only a broadcast bias add is recognised")
            bias_root = _bias_load(b[0])
            e = o[0]
        else:
            raise Unsupported(f"matmul epilogue op {e.name} is not recognised")
    acc_ok = e.kind == "matmul" or (e.kind == "opaque")
    if not acc_ok:
        raise Unsupported("the stored tile is not the matmul accumulator")
    if A.size1 != B.size0:
        raise ValueError("matmul: number of columns of lhs must be equal to number of rows of rhs")
    lo0, hi0 = _cover(tgt.start0, tgt.shape[0], L.ranges)
    lo1, hi1 = _cover(tgt.start1, tgt.shape[1], L.ranges)
    tl = _tensor_desc(A, L.args, lo0, hi0, 0, A.size1)
    tr = _tensor_desc(B, L.args, 0, B.size0, lo1, hi1)
    to = _tensor_desc(Cr, L.args, lo0, hi0, lo1, hi1)
    ep = abi.Epilogue(float(alpha), None, abi.F32, 1, activation, int(rounding))
    if bias_root is not None:
        root, axis = bias_root
        t = L.args[root.arg]
        esz = _ESZ[root.dtype]
        lo = lo1 if axis == 1 else lo0
        ep.bias = t.data_ptr() + (root.offset + lo * (root.stride1 if axis == 1 else root.stride0)) * esz
        ep.bias_dtype = root.dtype
        ep.bias_axis = axis
    way = int(L.matmuls[0].attrs.get("matmul_impl_way", 0))
    st = handle._lib.kapyb_matmul(handle._h, C.byref(tl), C.byref(tr), None, C.byref(to),
                                  C.byref(ep), way, sp)
    if st != abi.OK:
        handle._raise(st)
    return handle.last_kernel


def _is_splat_const(e: Expr) -> bool:
    while e.kind == "op" and e.name == "broadcast":
        e = e.args[0]
    return e.kind == "const"


def _splat_value(e: Expr) -> float:
    while e.kind == "op" and e.name == "broadcast":
        e = e.args[0]
    return float(e.value)


def _bias_load(e: Expr):
    """(root, axis) when `e` is broadcast(ld_global(row or column vector)) [+ extf]."""
    while e.kind == "op" and e.name in ("broadcast", "arith.extf"):
        e = e.args[0]
    if e.kind != "load":
        return None
    v = e.view
    if v.shape[0] == 1:
        return (v.root, 1)
    if v.shape[1] == 1:
        return (v.root, 0)
    return None
