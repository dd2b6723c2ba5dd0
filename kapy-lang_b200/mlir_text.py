"""Reader for the textual kapy IR: the custom assembly of the ops that appear on
the matmul / elementwise / reduce path (the syntax of
test/Conversion/KapyToKgpu/{matmul,elementwise_add,reduce_sum}.mlir, defined by
the assemblyFormat entries of include/kapy/Dialect/Kapy/IR/Ops.td).

It produces the same in-memory IR as ``ir.Builder``, so ``executor.launch`` runs
parsed kernels and built kernels alike.  It is a recogniser for this subset,
not an MLIR parser: anything outside the subset is a ``SyntaxError`` naming the
line.
"""
from __future__ import annotations

import re
from typing import Dict, List, Tuple

from . import ir

_ELEM = {"i1", "i8", "i16", "i32", "i64", "f16", "bf16", "f32", "f64"}
# MLIR's spellings of the two 8-bit float types (both E4M3 spellings reach the
# matmul as the finite-only format the MMA instruction reads)
_F8 = {"f8E4M3": "f8e4m3", "f8E4M3FN": "f8e4m3", "f8E5M2": "f8e5m2"}
_MEM = {"#global": ir.MemorySpace.GLOBAL_MEMORY, "#shared": ir.MemorySpace.SHARED_MEMORY,
        "#values": ir.MemorySpace.REGISTER_FILE}


def parse_type(text: str, aliases: Dict[str, ir.MemorySpace]):
    text = text.strip()
    if text in _ELEM:
        return ir.Type(text)
    if text in _F8:
        return ir.Type(_F8[text])
    if text.startswith("!kapy.ptr"):
        return ir.Type("ptr")
    m = re.fullmatch(r"tensor<([^,>]+?)(?:,\s*(#[\w.<>]+))?>", text)
    if not m:
        raise SyntaxError(f"unsupported type '{text}'")
    parts = m.group(1).split("x")
    elem = ir.Type(_F8.get(parts[-1].strip(), parts[-1].strip()))
    shape = tuple(-1 if p.strip() == "?" else int(p) for p in parts[:-1])
    enc = m.group(2)
    if enc is None:
        mem = ir.MemorySpace.REGISTER_FILE
    elif enc in aliases:
        mem = aliases[enc]
    else:
        mm = re.search(r"(global_memory|shared_memory|register_file)", enc)
        if not mm:
            raise SyntaxError(f"unknown encoding '{enc}'")
        mem = {"global_memory": ir.MemorySpace.GLOBAL_MEMORY,
               "shared_memory": ir.MemorySpace.SHARED_MEMORY,
               "register_file": ir.MemorySpace.REGISTER_FILE}[mm.group(1)]
    return ir.TensorType(shape, elem, mem)


def _split_top(text: str, sep: str = ",") -> List[str]:
    """Splits on `sep` outside <>, (), [] and {}."""
    out, depth, cur = [], 0, ""
    for ch in text:
        if ch in "<([{":
            depth += 1
        elif ch in ">)]}":
            depth -= 1
        if ch == sep and depth == 0:
            out.append(cur.strip())
            cur = ""
        else:
            cur += ch
    if cur.strip():
        out.append(cur.strip())
    return out


def _attr_dict(text: str) -> Dict[str, object]:
    out: Dict[str, object] = {}
    for item in _split_top(text.strip().strip("{}")):
        if "=" not in item:
            continue
        k, v = item.split("=", 1)
        v = v.split(":")[0].strip()
        if v in ("true", "false"):
            out[k.strip()] = v == "true"
        else:
            try:
                out[k.strip()] = int(v)
            except ValueError:
                out[k.strip()] = v
    return out


_FLOAT_OPS = {"arith.addf", "arith.subf", "arith.mulf", "arith.divf", "arith.remf",
              "arith.maximumf", "arith.minimumf", "arith.maxnumf", "arith.minnumf"}
_INT_OPS = {"arith.addi", "arith.subi", "arith.muli", "arith.divui", "arith.divsi", "arith.remui",
            "arith.remsi", "arith.andi", "arith.ori", "arith.xori", "arith.shli", "arith.shrui",
            "arith.shrsi", "arith.minsi", "arith.minui", "arith.maxsi", "arith.maxui"}
_UNARY = {"math.exp", "math.exp2", "math.log", "math.log2", "math.sqrt", "math.rsqrt", "math.erf",
          "math.sin", "math.cos", "math.floor", "math.ceil", "math.absf", "math.absi"}
_CASTS = {"arith.extf", "arith.truncf", "arith.sitofp", "arith.fptosi", "arith.bitcast",
          "arith.extsi", "arith.extui", "arith.trunci", "kapy.fptofp"}


class _Parser:
    def __init__(self, text: str, name: str = "<string>"):
        self.name = name
        self.lines = [re.sub(r"//.*$", "", ln).rstrip() for ln in text.splitlines()]
        self.pos = 0
        self.aliases: Dict[str, ir.MemorySpace] = dict(_MEM)
        self.module = ir.ModuleOp()

    def err(self, msg):
        return SyntaxError(f"{self.name}:{self.pos + 1}: {msg}")

    def ty(self, text):
        try:
            return parse_type(text, self.aliases)
        except SyntaxError as ex:
            raise self.err(str(ex))

    # ---------------------------------------------------------------- module
    def parse(self) -> ir.ModuleOp:
        while self.pos < len(self.lines):
            ln = self.lines[self.pos].strip()
            if not ln:
                self.pos += 1
            elif ln.startswith("#"):
                m = re.match(r"(#\w+)\s*=\s*#kapy\.encoding<(\w+)>", ln)
                if m:
                    self.aliases[m.group(1)] = {"global_memory": ir.MemorySpace.GLOBAL_MEMORY,
                                                "shared_memory": ir.MemorySpace.SHARED_MEMORY,
                                                "register_file": ir.MemorySpace.REGISTER_FILE}[
                        m.group(2)]
                self.pos += 1
            elif ln.startswith("module"):
                m = re.match(r"module(?:\s+attributes\s*(\{.*\}))?\s*\{$", ln)
                if not m:
                    raise self.err("malformed module header")
                if m.group(1):
                    self.module.attrs.update(_attr_dict(m.group(1)))
                self.pos += 1
            elif ln.startswith("kapy.func"):
                self.parse_func()
            elif ln == "}":
                self.pos += 1
            else:
                raise self.err(f"unexpected top-level text '{ln[:40]}'")
        return self.module

    def parse_func(self):
        ln = self.lines[self.pos].strip()
        m = re.match(r"kapy\.func\s+(?:(public|private)\s+)?@([\w.$-]+)\((.*)\)\s*(?:->\s*(.*?))?\s*\{$", ln)
        if not m:
            raise self.err("malformed kapy.func")
        vis, name, args = m.group(1) or "public", m.group(2), m.group(3)
        names, types, attrs = [], [], []
        for a in _split_top(args):
            am = re.match(r"(%[\w]+)\s*:\s*(.+?)(?:\s*(\{.*\}))?$", a)
            if not am:
                raise self.err(f"malformed argument '{a}'")
            names.append(am.group(1))
            types.append(self.ty(am.group(2)))
            attrs.append(_attr_dict(am.group(3)) if am.group(3) else {})
        results = tuple(self.ty(t) for t in _split_top(m.group(4).strip("()"))) if m.group(4) else ()
        func = ir.FuncOp(name, ir.FunctionType(tuple(types), results), vis, False)
        blk = func.add_entry_block()
        for i, d in enumerate(attrs):
            for k, v in d.items():
                func.set_arg_attr(i, k, v)
        env = {n: v for n, v in zip(names, blk.args)}
        for n, v in env.items():
            v.name = n
        self.pos += 1
        self.parse_block(blk, env)
        self.module.push_back(func)

    # ----------------------------------------------------------------- block
    def parse_block(self, blk: ir.Block, env: Dict[str, ir.Value]) -> str:
        """Parses ops until the closing '}' line; returns that line's tail."""
        while self.pos < len(self.lines):
            ln = self.lines[self.pos].strip()
            if not ln:
                self.pos += 1
                continue
            if ln.startswith("}"):
                self.pos += 1
                return ln[1:].strip()
            self.parse_op(ln, blk, env)
        raise self.err("unterminated region")

    def val(self, env, name):
        name = name.strip()
        if name not in env:
            raise self.err(f"use of undefined value {name}")
        return env[name]

    def add(self, blk, env, res_names, op: ir.Operation):
        op.parent_block = blk
        blk.ops.append(op)
        if res_names:
            if len(res_names) == 1 and ":" in res_names[0]:
                base, n = res_names[0].split(":")
                if int(n) != len(op.results):
                    raise self.err("result count mismatch")
                for i, r in enumerate(op.results):
                    env[f"{base}#{i}"] = r
                    r.name = f"{base}#{i}"
            else:
                if len(res_names) != len(op.results):
                    raise self.err(f"{op.name}: expected {len(op.results)} results")
                for n, r in zip(res_names, op.results):
                    env[n] = r
                    r.name = n
        return op

    def parse_op(self, ln: str, blk: ir.Block, env: Dict[str, ir.Value]):
        m = re.match(r"^(?:((?:%[\w#:]+\s*,\s*)*%[\w#:]+)\s*=\s*)?([a-z_]+\.[\w.]+)\s*(.*)$", ln)
        if not m:
            raise self.err(f"cannot parse '{ln[:60]}'")
        res = [r.strip() for r in m.group(1).split(",")] if m.group(1) else []
        name, rest = m.group(2), m.group(3)
        self.pos += 1
        V = lambda n: self.val(env, n)

        if name == "arith.constant":
            body, _, t = rest.rpartition(":")
            type_ = self.ty(t)
            body = body.strip()
            dm = re.match(r"dense<(.+)>", body)
            lit = dm.group(1) if dm else body
            if lit in ("true", "false"):
                value = lit == "true"
            else:
                value = float(lit) if ir.element_type(type_).is_float() else int(float(lit))
            return self.add(blk, env, res, ir.Operation(name, [], [type_], {"value": value}))
        if name in _FLOAT_OPS or name in _INT_OPS or name == "math.fma":
            ops, _, t = rest.rpartition(":")
            operands = [V(o) for o in _split_top(ops)]
            return self.add(blk, env, res, ir.Operation(name, operands, [self.ty(t)]))
        if name in _UNARY:
            ops, _, t = rest.rpartition(":")
            return self.add(blk, env, res, ir.Operation(name, [V(ops)], [self.ty(t)]))
        if name in ("arith.cmpi", "arith.cmpf"):
            ops, _, t = rest.rpartition(":")
            parts = _split_top(ops)
            src_t = self.ty(t)
            rt = (ir.TensorType(src_t.shape, ir.Type("i1"), src_t.memory)
                  if isinstance(src_t, ir.TensorType) else ir.Type("i1"))
            return self.add(blk, env, res, ir.Operation(name, [V(parts[1]), V(parts[2])], [rt],
                                                        {"predicate": parts[0]}))
        if name == "arith.select":
            # "%c, %a, %b : T" with a scalar condition, "... : tensor<..xi1>, T" with a
            # tensor of conditions: the result type is the last one
            ops, _, t = rest.partition(":")
            return self.add(blk, env, res,
                            ir.Operation(name, [V(o) for o in _split_top(ops)],
                                         [self.ty(_split_top(t)[-1])]))
        if name in _CASTS:
            mm = re.match(r"(%[\w#]+)\s*(\{.*\})?\s*:\s*(.+?)\s+to\s+(.+)$", rest)
            if not mm:
                raise self.err(f"malformed {name}")
            attrs = _attr_dict(mm.group(2)) if mm.group(2) else {}
            if "rounding_mode" in attrs:
                attrs["rounding_mode"] = ir.RoundingMode[str(attrs["rounding_mode"]).strip("#<>").split(" ")[-1].upper()] \
                    if not isinstance(attrs["rounding_mode"], int) else ir.RoundingMode(attrs["rounding_mode"])
            return self.add(blk, env, res, ir.Operation(name, [V(mm.group(1))], [self.ty(mm.group(4))], attrs))
        if name == "kapy.mk_global":
            mm = re.match(r"(%[\w#]+)\[(.+?)\]\s*\[(.+?)\]\s*\[(.+?)\]\s*:\s*(.+?)\s*->\s*(.+)$", rest)
            if not mm:
                raise self.err("malformed kapy.mk_global")
            sizes, strides = _split_top(mm.group(3)), _split_top(mm.group(4))
            operands = [V(mm.group(1)), V(mm.group(2)), V(sizes[0]), V(sizes[1]), V(strides[0]),
                        V(strides[1])]
            return self.add(blk, env, res, ir.Operation(name, operands, [self.ty(mm.group(6))]))
        if name in ("kapy.sv_global", "kapy.sv_shared"):
            mm = re.match(r"(%[\w#]+)\[(.+?):(.+?),(.+?):(.+?)\]\s*:\s*(.+?)\s*->\s*(.+)$", rest)
            if not mm:
                raise self.err(f"malformed {name}")
            operands = [V(mm.group(i)) for i in range(1, 6)]
            return self.add(blk, env, res, ir.Operation(name, operands, [self.ty(mm.group(7))]))
        if name == "kapy.ld_global":
            mm = re.match(r"(%[\w#]+)\s*(\{.*\})?\s*:\s*(.+?)\s*->\s*(.+)$", rest)
            if not mm:
                raise self.err("malformed kapy.ld_global")
            raw = _attr_dict(mm.group(2)) if mm.group(2) else {}
            attrs = {"padding_option": ir.PaddingOption.ZERO, "cache_modifier": ir.CacheModifier.NONE,
                     "evict_priority": ir.EvictPriority.EVICT_NORMAL,
                     "is_volatile": bool(raw.get("is_volatile", False))}
            if "padding_option" in raw:
                attrs["padding_option"] = ir.PaddingOption[str(raw["padding_option"]).strip("#<>").split(" ")[-1].upper()]
            return self.add(blk, env, res, ir.Operation(name, [V(mm.group(1))], [self.ty(mm.group(4))], attrs))
        if name == "kapy.st_global":
            ops, _, _t = rest.partition(":")
            ops = re.sub(r"\{.*\}", "", ops)
            return self.add(blk, env, res, ir.Operation(name, [V(o) for o in _split_top(ops)], [], {}))
        if name == "kapy.mk_shared":
            mm = re.match(r"(\{.*\})?\s*:\s*(.+)$", rest)
            attrs = _attr_dict(mm.group(1)) if mm and mm.group(1) else {}
            return self.add(blk, env, res, ir.Operation(name, [], [self.ty(mm.group(2))], attrs))
        if name == "kapy.cp_async_global_to_shared":
            ops = rest.split(":")[0]
            return self.add(blk, env, res, ir.Operation(name, [V(o) for o in _split_top(ops)], []))
        if name == "kapy.cp_async_wait_group":
            return self.add(blk, env, res, ir.Operation(name, [], [], _attr_dict(rest)))
        if name == "kapy.ld_matrix":
            mm = re.match(r"(.+?):\s*(.+)->\s*(.+)$", rest)
            return self.add(blk, env, res, ir.Operation(name, [V(o) for o in _split_top(mm.group(1))],
                                                        [self.ty(mm.group(3))]))
        if name == "kapy.matmul":
            mm = re.match(r"(\w+)\s+(.+?):\s*(.+)->\s*(.+)$", rest)
            if not mm:
                raise self.err("malformed kapy.matmul")
            way = ir.MatmulImplWay[mm.group(1).upper()]
            return self.add(blk, env, res, ir.Operation(name, [V(o) for o in _split_top(mm.group(2))],
                                                        [self.ty(mm.group(4))], {"matmul_impl_way": way}))
        if name == "kapy.program_id":
            mm = re.match(r"(\{.*\})\s*:\s*(.+)$", rest)
            return self.add(blk, env, res, ir.Operation(name, [], [self.ty(mm.group(2))],
                                                        {"axis": int(_attr_dict(mm.group(1))["axis"])}))
        if name in ("kapy.warp_id", "kapy.lane_id"):
            return self.add(blk, env, res, ir.Operation(name, [], [self.ty(rest.lstrip(": "))]))
        if name in ("kapy.splat", "kapy.broadcast", "kapy.transpose"):
            mm = re.match(r"(%[\w#]+)\s*:\s*(.+?)\s*->\s*(.+)$", rest)
            return self.add(blk, env, res, ir.Operation(name, [V(mm.group(1))], [self.ty(mm.group(3))]))
        if name == "kapy.clampf":
            mm = re.match(r"(.+?)(\{.*\})?\s*:\s*(.+)$", rest)
            attrs = _attr_dict(mm.group(2)) if mm.group(2) else {}
            return self.add(blk, env, res, ir.Operation(name, [V(o) for o in _split_top(mm.group(1))],
                                                        [self.ty(mm.group(3))],
                                                        {"propagate_nan": bool(attrs.get("propagate_nan", False))}))
        if name == "kapy.return":
            ops = rest.split(":")[0].strip()
            return self.add(blk, env, res, ir.Operation(name, [V(o) for o in _split_top(ops)] if ops else [], []))
        if name == "scf.yield":
            ops = rest.split(":")[0].strip()
            return self.add(blk, env, res, ir.Operation(name, [V(o) for o in _split_top(ops)] if ops else [], []))
        if name == "kapy.reduce":
            mm = re.match(r"(%[\w#]+)\s*(\{.*?\})\s*lambda\((.*)\)\s*\{$", rest)
            if not mm:
                raise self.err("malformed kapy.reduce")
            op = ir.Operation(name, [V(mm.group(1))], [], {"axis": int(_attr_dict(mm.group(2))["axis"])},
                              n_regions=1)
            body = ir.Block()
            body.parent_op = op
            inner = dict(env)
            for a in _split_top(mm.group(3)):
                an, at = a.split(":")
                v = body.add_argument(self.ty(at))
                v.name = an.strip()
                inner[an.strip()] = v
            op.regions[0].blocks.append(body)
            tail = self.parse_block(body, inner)
            tm = re.match(r":\s*(.+?)\s*->\s*(.+)$", tail)
            if not tm:
                raise self.err("kapy.reduce: missing result type")
            op.results = [ir.Value(self.ty(tm.group(2)), op, 0)]
            return self.add(blk, env, res, op)
        if name == "scf.for":
            mm = re.match(r"(%[\w]+)\s*=\s*(%[\w#]+)\s+to\s+(%[\w#]+)\s+step\s+(%[\w#]+)"
                          r"(?:\s+iter_args\((.*?)\)\s*->\s*\((.*?)\))?\s*(?::\s*(\w+))?\s*\{$", rest)
            if not mm:
                raise self.err("malformed scf.for")
            iv_name = mm.group(1)
            inits, names = [], []
            if mm.group(5):
                for a in _split_top(mm.group(5)):
                    an, init = a.split("=")
                    names.append(an.strip())
                    inits.append(V(init))
            rtypes = [self.ty(t) for t in _split_top(mm.group(6))] if mm.group(6) else []
            lb, ub, step = V(mm.group(2)), V(mm.group(3)), V(mm.group(4))
            op = ir.Operation(name, [lb, ub, step, *inits], rtypes, n_regions=1)
            body = ir.Block([lb.type, *rtypes])
            body.parent_op = op
            op.regions[0].blocks.append(body)
            inner = dict(env)
            inner[iv_name] = body.args[0]
            body.args[0].name = iv_name
            for n, v in zip(names, body.args[1:]):
                inner[n] = v
                v.name = n
            self.parse_block(body, inner)
            return self.add(blk, env, res, op)
        raise self.err(f"op '{name}' is outside the recognised subset")


def parse_text(text: str, name: str = "<string>") -> ir.ModuleOp:
    return _Parser(text, name).parse()


def parse_file(path: str) -> ir.ModuleOp:
    with open(path) as f:
        return parse_text(f.read(), path)
