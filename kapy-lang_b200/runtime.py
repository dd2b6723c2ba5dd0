"""Host-side runtime: a `Handle` per GPU that turns torch tensors (device memory
and streams are torch's job) into the descriptors of ``include/kapyb.h`` and
calls the C ABI.  Errors come back as the exception classes the reference's
bindings raise: ``ValueError`` for verifier-style rejections (the reference
raises ``std::invalid_argument`` / fails ``verify()``), ``RuntimeError`` for
everything else (``std::runtime_error("pass manager run failed")``,
python/src/passes.cc:72-75).
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Optional, Sequence

from . import _abi as abi


class KapybError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"kapyb status {status}: {message}")
        self.status = status


class KapybTimeout(KapybError):
    pass


def _torch():
    import torch
    return torch


def dtype_code(dt) -> int:
    torch = _torch()
    if dt == torch.float16:
        return abi.F16
    if dt == torch.bfloat16:
        return abi.BF16
    if dt == torch.float32:
        return abi.F32
    if dt == torch.float8_e4m3fn:
        return abi.F8E4M3
    if dt == torch.float8_e5m2:
        return abi.F8E5M2
    raise ValueError(f"unsupported element type {dt}")


def torch_dtype(code: int):
    torch = _torch()
    return {abi.F16: torch.float16, abi.BF16: torch.bfloat16, abi.F32: torch.float32,
            abi.F8E4M3: torch.float8_e4m3fn, abi.F8E5M2: torch.float8_e5m2}[code]


def tensor2d(t, padding: int = abi.PAD_ZERO, cache: int = 0) -> abi.Tensor2d:
    """kapy.mk_global over a 2-D torch tensor (any strides that fit i32).  `cache`:
    abi.cache_hints(...) of the ld_global / st_global that touches the tensor."""
    if t.dim() != 2:
        raise ValueError("kapy tensors are rank 2")
    s0, s1 = t.stride()
    for v in (t.shape[0], t.shape[1], s0, s1):
        if v >= 2 ** 31:
            raise ValueError("sizes and strides must fit i32")
    return abi.Tensor2d(t.data_ptr(), 0, t.shape[0], t.shape[1], s0, s1, dtype_code(t.dtype),
                        padding, int(cache), 0)


def matmul_plan(m: int, n: int, k: int, *, dtype=abi.BF16, rhs_dtype=None, out_dtype=None,
                lhs_strides=None, rhs_strides=None, out_strides=None, batch: int = 1,
                sm_count: int = 148, align: int = 256, handle=None) -> str:
    """Text of kapyb_matmul_plan for an [m,k] x [k,n] problem described by shape,
    strides (elements; row-major by default) and the byte alignment of its base
    addresses.  Needs no GPU unless a handle is given."""
    lib = abi.load()
    rhs_dtype = dtype if rhs_dtype is None else rhs_dtype
    out_dtype = dtype if out_dtype is None else out_dtype

    def desc(rows, cols, strides, dt):
        s0, s1 = strides if strides is not None else (cols, 1)
        return abi.Tensor2d(align, 0, rows, cols, s0, s1, dt, abi.PAD_ZERO)

    tl, tr, to = desc(m, k, lhs_strides, dtype), desc(k, n, rhs_strides, rhs_dtype), \
        desc(m, n, out_strides, out_dtype)
    buf = C.create_string_buffer(2048)
    st = lib.kapyb_matmul_plan(handle._h if handle is not None else None,
                               0 if handle is not None else int(sm_count), C.byref(tl),
                               C.byref(tr), C.byref(to), int(batch), buf, len(buf))
    if st != abi.OK:
        msg = lib.kapyb_last_error_string(handle._h if handle is not None else None).decode()
        if st == abi.INVALID_ARG:
            raise ValueError(msg)
        raise KapybError(st, msg)
    return buf.value.decode()


_DTYPE_NAMES = {abi.F16: "f16", abi.BF16: "bf16", abi.F32: "f32", abi.F8E4M3: "f8E4M3",
                abi.F8E5M2: "f8E5M2"}


def tuning_load(path: str) -> int:
    """Adds the tuned dispatch choices of a file to the process-wide table."""
    n = C.c_int32(0)
    lib = abi.load()
    st = lib.kapyb_tuning_load(os.fsencode(path), C.byref(n))
    if st != abi.OK:
        raise ValueError(lib.kapyb_last_error_string(None).decode())
    return n.value


def tuning_clear() -> None:
    abi.load().kapyb_tuning_clear()


def tune_matmul(handle, lhs, rhs, out=None, *, file: Optional[str] = None, iters: int = 10,
                candidates: Optional[Sequence[str]] = None, **epilogue):
    """Times the kernel families on this very problem (device tensors, 2-D or
    batched 3-D) and returns (best path, {path: seconds}).  With `file`, appends
    the winner as a line kapyb_tuning_load understands."""
    torch = _torch()
    batched = lhs.dim() == 3
    m, k = lhs.shape[-2], lhs.shape[-1]
    n = rhs.shape[-1]
    if candidates is None:
        candidates = ["auto", "1cta:64", "1cta:128", "1cta:256", "2cta:128", "2cta:256", "2cta:512"]
        if m <= 64 and not batched:
            candidates.append("skinny")
    if out is None:
        out = torch.empty(lhs.shape[:-1] + (n,), device=lhs.device,
                          dtype=torch.bfloat16 if lhs.dtype.itemsize == 1 else lhs.dtype)
    times = {}
    # what the dispatcher's own choice computes: a forced family has to reproduce it
    handle.set_matmul_path("auto")
    handle.matmul(lhs, rhs, out, **epilogue)
    handle.check()
    want = out.clone()
    try:
        for path in candidates:
            try:
                handle.set_matmul_path(path)
                out.zero_()
                for _ in range(3):
                    handle.matmul(lhs, rhs, out, **epilogue)
                handle.check()
            except (KapybError, ValueError):
                continue  # this family does not take the problem
            # families differ in summation order only: a candidate whose result is off
            # by more than that is broken for this problem and must not win
            d = (out.float() - want.float()).abs().max().item()
            scale = want.float().abs().max().item() or 1.0
            if not (d <= 2e-2 * scale):
                continue
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(iters):
                handle.matmul(lhs, rhs, out, **epilogue)
            e1.record()
            e1.synchronize()
            times[path] = e0.elapsed_time(e1) * 1e-3 / iters
    finally:
        handle.set_matmul_path("auto")
    best = min(times, key=times.get)
    if file is not None and best != "auto":
        la, lb = (lhs[0], rhs[0]) if batched else (lhs, rhs)
        lo = out[0] if batched else out
        # The table is keyed by the problem as the kernel sees it.  An output with
        # its unit stride on axis 0 is computed as the transposed problem
        # (C^T = B^T . A^T): M and N swap, and so do the operands and their majors.
        a_k = la.stride(1) == 1 or k == 1
        b_n = lb.stride(1) == 1 or n == 1
        if lo.stride(1) != 1 and lo.stride(0) == 1:
            m, n = n, m
            a_k, b_n = (lb.stride(0) == 1 or k == 1), (la.stride(0) == 1 or n == 1)
        amaj = "k" if a_k else "mn"
        bmaj = "mn" if b_n else "k"
        with open(file, "a") as f:
            f.write(f"{m} {n} {k} {lhs.shape[0] if batched else 1} {_DTYPE_NAMES[dtype_code(lhs.dtype)]} "
                    f"{amaj} {bmaj} {best}  # {times[best] * 1e6:.1f} us, auto {times.get('auto', 0) * 1e6:.1f} us\n")
    return best, times


class Handle:
    """One per (thread, GPU).  Owns the library context; tensors stay the caller's."""

    def __init__(self, device: int = 0):
        self._lib = abi.load()
        self._h = C.c_void_p()
        st = self._lib.kapyb_create(C.byref(self._h), int(device))
        if st != abi.OK:
            msg = self._lib.kapyb_last_error_string(None).decode()
            raise KapybError(st, msg)
        self.device = int(device)

    def close(self):
        if getattr(self, "_h", None) is not None and self._h:
            self._lib.kapyb_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # ------------------------------------------------------------ utilities
    def _raise(self, st: int):
        msg = self._lib.kapyb_last_error_string(self._h).decode()
        if st == abi.INVALID_ARG:
            raise ValueError(msg)
        if st == abi.TIMEOUT:
            raise KapybTimeout(st, msg)
        raise KapybError(st, msg)

    def _stream(self, stream=None) -> C.c_void_p:
        if stream is None:
            stream = _torch().cuda.current_stream(self.device)
        return C.c_void_p(getattr(stream, "cuda_stream", stream))

    def check(self, stream=None):
        """Synchronises the stream and raises if a kernel reported a timeout."""
        st = self._lib.kapyb_check(self._h, self._stream(stream))
        if st != abi.OK:
            self._raise(st)

    def reserve_workspace(self, nbytes: int):
        st = self._lib.kapyb_reserve_workspace(self._h, int(nbytes))
        if st != abi.OK:
            self._raise(st)

    @property
    def last_kernel(self) -> str:
        return self._lib.kapyb_last_kernel(self._h).decode()

    @property
    def launch_count(self) -> int:
        return int(self._lib.kapyb_launch_count(self._h))

    def probe_read(self, n: int = 2, stream=None):
        """Probe words of the last matmul run with debug bit 7 (":d128")."""
        words = (C.c_uint32 * 14)()
        st = self._lib.kapyb_probe_read(self._h, self._stream(stream), words, n)
        if st != abi.OK:
            self._raise(st)
        return [int(w) for w in words[:n]]

    def probe_clock(self, stream=None):
        """(cycles, nanoseconds) of the last matmul run with debug bit 7 (":d128")."""
        cyc, ns = self.probe_read(2, stream)
        return cyc, ns

    def set_matmul_path(self, name: str):
        st = self._lib.kapyb_set_matmul_path(self._h, name.encode())
        if st != abi.OK:
            self._raise(st)

    def _epilogue(self, alpha, bias, bias_axis, activation, rounding):
        ep = abi.Epilogue(float(alpha), None, abi.F32, int(bias_axis), int(activation),
                          int(rounding))
        if bias is not None:
            if not bias.is_contiguous():
                raise ValueError("bias must be contiguous")
            ep.bias = bias.data_ptr()
            ep.bias_dtype = dtype_code(bias.dtype)
        return ep

    # --------------------------------------------------------------- matmul
    def matmul(self, lhs, rhs, out=None, *, acc=None, alpha: float = 1.0, bias=None,
               bias_axis: int = 1, activation: int = abi.ACT_NONE, rounding: int = abi.RN,
               out_dtype=None, impl_way: int = abi.MMA_ANY, stream=None,
               cache=(0, 0, 0)):
        """kapy.matmul at whole-problem scope; 3-D operands run as a batch.  `cache`:
        abi.cache_hints(...) for lhs, rhs and out (their eviction priority becomes the
        L2 policy of the tile loads / stores)."""
        torch = _torch()
        if lhs.dim() == 3:
            return self._matmul_batched(lhs, rhs, out, alpha=alpha, bias=bias, bias_axis=bias_axis,
                                        activation=activation, rounding=rounding,
                                        out_dtype=out_dtype, impl_way=impl_way, stream=stream)
        if out is None:
            out = torch.empty((lhs.shape[0], rhs.shape[1]), device=lhs.device,
                              dtype=out_dtype or lhs.dtype)
        tl, tr, to = tensor2d(lhs, cache=cache[0]), tensor2d(rhs, cache=cache[1]), \
            tensor2d(out, cache=cache[2])
        ta = tensor2d(acc) if acc is not None else None
        ep = self._epilogue(alpha, bias, bias_axis, activation, rounding)
        st = self._lib.kapyb_matmul(self._h, C.byref(tl), C.byref(tr),
                                    C.byref(ta) if ta is not None else None, C.byref(to),
                                    C.byref(ep), impl_way, self._stream(stream))
        if st != abi.OK:
            self._raise(st)
        return out

    def matmul_reduce(self, lhs, rhs, axis: int, out=None, reduced=None, *, alpha: float = 1.0,
                      bias=None, bias_axis: int = 1, activation: int = abi.ACT_NONE,
                      rounding: int = abi.RN, out_dtype=None, combiner: int = abi.RED_ADD,
                      impl_way: int = abi.MMA_ANY, stream=None):
        """matmul whose epilogue also sums its f32 result along `axis` (kapy.reduce
        with an addf lambda on the accumulator tile).  Returns (out, reduced)."""
        torch = _torch()
        if out is None:
            out = torch.empty((lhs.shape[0], rhs.shape[1]), device=lhs.device,
                              dtype=out_dtype or lhs.dtype)
        if reduced is None:
            shape = (1, rhs.shape[1]) if axis == 0 else (lhs.shape[0], 1)
            reduced = torch.empty(shape, device=lhs.device, dtype=torch.float32)
        tl, tr, to, td = tensor2d(lhs), tensor2d(rhs), tensor2d(out), tensor2d(reduced)
        ep = self._epilogue(alpha, bias, bias_axis, activation, rounding)
        st = self._lib.kapyb_matmul_reduce(self._h, C.byref(tl), C.byref(tr), C.byref(to),
                                           C.byref(td), int(axis), int(combiner), C.byref(ep),
                                           impl_way, self._stream(stream))
        if st != abi.OK:
            self._raise(st)
        return out, reduced

    def _matmul_batched(self, lhs, rhs, out, *, alpha, bias, bias_axis, activation, rounding,
                        out_dtype, impl_way, stream):
        torch = _torch()
        if rhs.dim() != 3 or rhs.shape[0] != lhs.shape[0]:
            raise ValueError("batched matmul needs [B,M,K] and [B,K,N]")
        B = lhs.shape[0]
        if out is None:
            out = torch.empty((B, lhs.shape[1], rhs.shape[2]), device=lhs.device,
                              dtype=out_dtype or lhs.dtype)
        tl, tr, to = tensor2d(lhs[0]), tensor2d(rhs[0]), tensor2d(out[0])
        ep = self._epilogue(alpha, bias, bias_axis, activation, rounding)
        st = self._lib.kapyb_matmul_batched(self._h, C.byref(tl), C.byref(tr), C.byref(to), B,
                                            lhs.stride(0), rhs.stride(0), out.stride(0),
                                            C.byref(ep), impl_way, self._stream(stream))
        if st != abi.OK:
            self._raise(st)
        return out

    def matmul_host(self, lhs, rhs, out, *, alpha: float = 1.0, bias=None, bias_axis: int = 1,
                    activation: int = abi.ACT_NONE, rounding: int = abi.RN,
                    impl_way: int = abi.MMA_ANY, stream=None):
        """Same call on CPU tensors (pinned or pageable): copies in, computes on
        the GPU, copies `out` back, returns when it has landed."""
        for t in (lhs, rhs, out):
            if t.is_cuda:
                raise ValueError("matmul_host takes host tensors")
        tl, tr, to = tensor2d(lhs), tensor2d(rhs), tensor2d(out)
        ep = self._epilogue(alpha, bias, bias_axis, activation, rounding)
        st = self._lib.kapyb_matmul_host(self._h, C.byref(tl), C.byref(tr), C.byref(to),
                                         C.byref(ep), impl_way, self._stream(stream))
        if st != abi.OK:
            self._raise(st)
        return out

    def matmul_push(self, lhs, rhs_shard, peer_ptrs: Sequence[int], *, out_dtype, out_stride0: int,
                    col_begin: int, n_total: int, alpha: float = 1.0, bias=None,
                    activation: int = abi.ACT_NONE, rounding: int = abi.RN,
                    impl_way: int = abi.MMA_ANY, stream=None):
        """N-sharded matmul whose epilogue stores this rank's column block into
        every peer's full-size output (device pointers in `peer_ptrs`)."""
        tl, tr = tensor2d(lhs), tensor2d(rhs_shard)
        ep = self._epilogue(alpha, bias, 1, activation, rounding)
        arr = (C.c_void_p * len(peer_ptrs))(*[C.c_void_p(p) for p in peer_ptrs])
        st = self._lib.kapyb_matmul_push(self._h, C.byref(tl), C.byref(tr), arr, len(peer_ptrs),
                                         dtype_code(out_dtype), out_stride0, col_begin, n_total,
                                         C.byref(ep), impl_way, self._stream(stream))
        if st != abi.OK:
            self._raise(st)

    def gather_signal(self, peer_flag_ptrs: Sequence[int], my_rank: int, seq: int, stream=None):
        """Stores `seq` into word `my_rank` of every rank's flag array (device
        pointers), ordered after the work already on the stream."""
        arr = (C.c_void_p * len(peer_flag_ptrs))(*[C.c_void_p(p) for p in peer_flag_ptrs])
        st = self._lib.kapyb_gather_signal(self._h, arr, len(peer_flag_ptrs), int(my_rank),
                                           int(seq) & 0xFFFFFFFF, self._stream(stream))
        if st != abi.OK:
            self._raise(st)

    def gather_wait(self, my_flags_ptr: int, n_ranks: int, seq: int, limit_ms: int = 0,
                    stream=None):
        """Stream-ordered, bounded wait until every word of this rank's flag array
        has reached `seq`; a time-out surfaces in check()."""
        st = self._lib.kapyb_gather_wait(self._h, C.c_void_p(my_flags_ptr), int(n_ranks),
                                         int(seq) & 0xFFFFFFFF, int(limit_ms), self._stream(stream))
        if st != abi.OK:
            self._raise(st)

    def matmul_host_sharded(self, lhs_rows, m_total: int, row_begin: int, rhs, out, *,
                            peer_lhs_ptrs: Sequence[int], peer_flag_ptrs: Sequence[int], rank: int,
                            seq: int, wait_limit_ms: int = 0, alpha: float = 1.0, bias=None,
                            bias_axis: int = 1, activation: int = abi.ACT_NONE,
                            rounding: int = abi.RN, impl_way: int = abi.MMA_ANY, stream=None):
        """Host tensors in, host tensor out, on `len(peer_lhs_ptrs)` GPUs: this
        rank uploads rows [row_begin, row_begin + len(lhs_rows)) of lhs and its
        column block `rhs` of B, receives the other rows from its peers over
        NVLink, and computes out = lhs . rhs (see kapyb_matmul_host_sharded)."""
        for t in (lhs_rows, rhs, out):
            if t.is_cuda:
                raise ValueError("matmul_host_sharded takes host tensors")
        world = len(peer_lhs_ptrs)
        tl, tr, to = tensor2d(lhs_rows), tensor2d(rhs), tensor2d(out)
        ep = self._epilogue(alpha, bias, bias_axis, activation, rounding)
        pl = (C.c_void_p * world)(*[C.c_void_p(p) for p in peer_lhs_ptrs])
        pf = (C.c_void_p * world)(*[C.c_void_p(p) for p in peer_flag_ptrs])
        ctx = abi.ShardCtx(int(rank), world, pl, pf, int(seq) & 0xFFFFFFFF, int(wait_limit_ms))
        st = self._lib.kapyb_matmul_host_sharded(self._h, C.byref(tl), int(m_total), int(row_begin),
                                                 C.byref(tr), C.byref(to), C.byref(ep),
                                                 C.byref(ctx), impl_way, self._stream(stream))
        if st != abi.OK:
            self._raise(st)
        return out

    # ---------------------------------------------------- elementwise/reduce
    def elementwise(self, insts, inputs, out, paddings: Optional[Sequence[int]] = None,
                    stream=None, caches: Optional[Sequence[int]] = None, out_cache: int = 0):
        """Runs a recorded op list [(op,dtype,dst,a,b,c,imm,flags), ...].  `caches` /
        `out_cache`: abi.cache_hints(...) per input / for the output."""
        prog = (abi.Inst * max(1, len(insts)))()
        for i, t in enumerate(insts):
            prog[i] = abi.Inst(*t)
        tin = (abi.Tensor2d * max(1, len(inputs)))()
        for i, t in enumerate(inputs):
            tin[i] = tensor2d(t, paddings[i] if paddings else abi.PAD_ZERO,
                              caches[i] if caches else 0)
        to = tensor2d(out, cache=out_cache)
        st = self._lib.kapyb_elementwise(self._h, prog, len(insts), tin, len(inputs),
                                         C.byref(to), self._stream(stream))
        if st != abi.OK:
            self._raise(st)
        return out

    def reduce(self, src, axis: int, combiner: int = abi.RED_ADD, out=None, out_dtype=None,
               stream=None):
        """kapy.reduce along `axis` of a 2-D tensor; the reduced axis becomes 1."""
        torch = _torch()
        if out is None:
            shape = (1, src.shape[1]) if axis == 0 else (src.shape[0], 1)
            out = torch.empty(shape, device=src.device, dtype=out_dtype or src.dtype)
        ts, td = tensor2d(src), tensor2d(out)
        st = self._lib.kapyb_reduce(self._h, C.byref(ts), C.byref(td), int(axis), int(combiner),
                                    self._stream(stream))
        if st != abi.OK:
            self._raise(st)
        return out


def shard_range(total: int, parts: int, rank: int, align: int = 1):
    """[begin, end) of `total` units owned by `rank` (blocks of `align`)."""
    lib = abi.load()
    b, e = C.c_int64(), C.c_int64()
    st = lib.kapyb_shard_range(total, parts, rank, align, C.byref(b), C.byref(e))
    if st != abi.OK:
        raise ValueError("bad shard arguments")
    return int(b.value), int(e.value)
