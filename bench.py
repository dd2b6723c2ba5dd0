#!/usr/bin/env python
"""Benchmark of the hot path: bf16 GEMM M=N=K=8192, row-major A/B, fp32
accumulate, bf16 output with a fused per-column bias (synthetic inputs,
normal(0, 1/sqrt(K)) from a seed; bias uniform[-0.1, 0.1]).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

One step = one pass of the hot path over the whole problem.  N > 1 (under
torchrun) shards the columns of B and of the output across ranks with no
collective on the data path; the fused push all-gather is timed separately and
reported under "gather".  Rank 0 prints one JSON line.

`--impl reference` times the reference's arithmetic on the host cores (the CPU
restatement under oracle/, since the reference itself stops at a PTX string and
has no executable path) on a bounded row sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

M = N = K = 8192
SEED = 1002
METRIC = "bf16_gemm_tflops"
UNIT = "TFLOP/s"
FLOPS = 2.0 * M * N * K                       # algorithmic FLOPs of one step
ALG_BYTES = 3 * M * N * 2 + N * 2             # A + B + C (bf16) + bias
CPU_SAMPLE_ROWS = 512                         # rows of the output the CPU arm computes per step
# dram__bytes_read.sum + dram__bytes_write.sum of one full-size launch of the
# dominant kernel, from a one-pass ncu capture of this benchmark (command and
# figures in profiles/gemm_tcgen05_2cta_256x512_bf16_8192x8192x4096.txt).
NCU_TRAFFIC_BYTES = 869_611_008 + 151_768_576


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"bf16_burst": p["bf16_tflops"], "bf16_sustained": p["bf16_tflops_sustained"],
                "hbm_gbs": p["hbm_gbs"], "source": "measured"}
    return {"bf16_burst": 1590.0, "bf16_sustained": 1400.0, "hbm_gbs": 6650.0,
            "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons through NVML (read-only queries)
    from a thread while the timed region runs."""

    def __init__(self, index: int):
        self.index = index
        self.samples = []
        self._stop = threading.Event()
        self.thread = None
        self.err = None

    def _run(self):
        try:
            import pynvml as nv
            nv.nvmlInit()
            uuid = None
            try:
                import torch
                uuid = str(torch.cuda.get_device_properties(self.index).uuid)
            except Exception:
                pass
            hdl = None
            if uuid:
                for cand in (uuid, "GPU-" + uuid):
                    try:
                        hdl = nv.nvmlDeviceGetHandleByUUID(cand.encode())
                        break
                    except Exception:
                        continue
            if hdl is None:
                hdl = nv.nvmlDeviceGetHandleByIndex(self.index)
            self.max_mhz = nv.nvmlDeviceGetMaxClockInfo(hdl, nv.NVML_CLOCK_SM)
            while not self._stop.is_set():
                mhz = nv.nvmlDeviceGetClockInfo(hdl, nv.NVML_CLOCK_SM)
                try:
                    reasons = nv.nvmlDeviceGetCurrentClocksEventReasons(hdl)
                except Exception:
                    reasons = nv.nvmlDeviceGetCurrentClocksThrottleReasons(hdl)
                self.samples.append((time.perf_counter(), mhz, reasons))
                time.sleep(0.002)
        except Exception as ex:  # NVML missing: report it, do not fail the run
            self.err = repr(ex)

    def start(self):
        self.thread = threading.Thread(target=self._run, daemon=True)
        self.thread.start()
        # NVML's first call can take a while: wait for the first sample
        t0 = time.perf_counter()
        while not self.samples and self.err is None and time.perf_counter() - t0 < 3.0:
            time.sleep(0.01)

    def stop(self, t_begin=None, t_end=None):
        self._stop.set()
        if self.thread is not None:
            self.thread.join(timeout=5)
        rows = [s for s in self.samples
                if (t_begin is None or s[0] >= t_begin) and (t_end is None or s[0] <= t_end)]
        if not rows:
            rows = self.samples[-3:]
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [self.err or "no samples"]}
        bits = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown",
                0x4: "sw_power_cap"}
        seen = set()
        for _, _, r in rows:
            for b, name in bits.items():
                if r & b:
                    seen.add(name)
        return {"sm_mhz": statistics.median(m for _, m, _ in rows),
                "sm_max_mhz": getattr(self, "max_mhz", None), "reasons": sorted(seen),
                "samples": len(rows)}


def make_inputs(torch, n_cols_begin=0, n_cols_end=N):
    """Seeded host tensors (pinned).  Every rank draws the full B so that shards
    are slices of the same matrix whatever the world size."""
    g = torch.Generator(device="cpu").manual_seed(SEED)
    A = (torch.randn(M, K, generator=g) * K ** -0.5).to(torch.bfloat16)
    B = (torch.randn(K, N, generator=g) * K ** -0.5).to(torch.bfloat16)
    bias = (torch.rand(N, generator=g) * 0.2 - 0.1).to(torch.bfloat16)
    B = B[:, n_cols_begin:n_cols_end].contiguous()
    bias = bias[n_cols_begin:n_cols_end].contiguous()
    return A, B, bias


def cpu_step(ko, A_bits, B_bits, bias_bits, rows):
    return ko.matmul_f32acc(A_bits, ko.BF16, B_bits, ko.BF16, ko.BF16, bias=bias_bits,
                            bias_dtype=ko.BF16, row_begin=0, row_end=rows)


def run_reference(args):
    """Reference arm: the path's arithmetic on the host cores (rank 0 only)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import numpy as np
    import torch

    import oracle as ko
    ko.build()
    A, B, bias = make_inputs(torch)
    bits = lambda t: t.view(torch.int16).numpy().view(np.uint16)
    Ab, Bb, bb = bits(A), bits(B), bits(bias)
    rows = CPU_SAMPLE_ROWS
    for _ in range(max(1, min(args.warmup, 1))):
        cpu_step(ko, Ab, Bb, bb, 32)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_step(ko, Ab, Bb, bb, rows)
    dt = (time.perf_counter() - t0) / args.steps
    value = 2.0 * rows * N * K / dt / 1e12
    cores = ko.num_threads()
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT,
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "bf16 GEMM M=N=K=8192 row-major A/B, fp32 accumulate, bf16 out, "
                               "fused per-column bias", "seed": SEED},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port",
                         "sample": f"rows [0,{rows}) of the {M}x{N} output per step "
                                   f"(all of B and K), OpenMP on {cores} threads"},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


def secondary(torch, pkg, h, peaks):
    """The other single-GPU configurations, timed with the same hygiene (inputs
    larger than L2 or L2 flushed between iterations), for context."""
    out = {}
    abi = pkg.abi
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")

    def timeit(fn, iters=10, flush_l2=False):
        """Median over 5 samples of `iters` back-to-back launches (one event pair
        per sample), or of single launches with an L2 flush before each when the
        working set would otherwise stay in L2."""
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        ts = []
        for _ in range(5 if not flush_l2 else iters):
            if flush_l2:
                flush.zero_()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            for _ in range(1 if flush_l2 else iters):
                fn()
            e.record()
            e.synchronize()
            ts.append(s.elapsed_time(e) * 1e-3 / (1 if flush_l2 else iters))
        return statistics.median(ts)

    g = torch.Generator(device="cpu").manual_seed(1003)
    n = 1 << 28
    x = torch.randn(1 << 24, generator=g).to(torch.bfloat16).cuda().repeat(16).view(1, n)
    y = torch.empty_like(x)
    prog = pkg.programs.affine_gelu_tanh(abi.BF16, 0.5, 0.1)
    t = timeit(lambda: h.elementwise(prog, [x], y))
    gbs = n * 4 / t / 1e9
    out["gelu_tanh_affine_2^28_bf16"] = {"GB/s": gbs, "frac_of_measured_hbm": gbs / peaks["hbm_gbs"],
                                         "ms": t * 1e3, "kernel": h.last_kernel}
    prog_lin = pkg.programs.affine(abi.BF16, 0.5, 0.1)
    t = timeit(lambda: h.elementwise(prog_lin, [x], y))
    gbs = n * 4 / t / 1e9
    out["affine_2^28_bf16"] = {"GB/s": gbs, "frac_of_measured_hbm": gbs / peaks["hbm_gbs"],
                               "ms": t * 1e3, "kernel": h.last_kernel}
    del y
    X = x.view(65536, 4096)
    s = torch.empty((65536, 1), dtype=torch.float32, device="cuda")
    t = timeit(lambda: h.reduce(X, axis=1, out=s))
    gbs = (65536 * 4096 * 2 + 65536 * 4) / t / 1e9
    out["rowsum_65536x4096_bf16"] = {"GB/s": gbs, "frac_of_measured_hbm": gbs / peaks["hbm_gbs"],
                                     "ms": t * 1e3, "kernel": h.last_kernel}
    del x, X, s
    # decode shape: M=16, N=28672, K=8192 (weights 470 MB > L2)
    Xs = torch.randn(16, 8192, generator=g).to(torch.bfloat16).cuda()
    W = (torch.randn(8192, 28672 // 8, generator=g) * 0.02).to(torch.bfloat16).cuda().repeat(1, 8)
    o = torch.empty((16, 28672), dtype=torch.bfloat16, device="cuda")
    t = timeit(lambda: h.matmul(Xs, W, out=o))
    gbs = 470941696 / t / 1e9
    out["decode_16x28672x8192_bf16"] = {"GB/s": gbs, "frac_of_measured_hbm": gbs / peaks["hbm_gbs"],
                                        "ms": t * 1e3, "kernel": h.last_kernel}
    # the vendor library on the same buffers, for context only (not on the product path)
    t_lib = timeit(lambda: torch.mm(Xs, W, out=o))
    out["decode_16x28672x8192_bf16"]["library_torch_mm_GB/s"] = 470941696 / t_lib / 1e9
    del W, o
    # attention-score shape: batch 64 x 2048 x 2048 x 128, alpha = 1/sqrt(128)
    Q = torch.randn(8, 2048, 128, generator=g).to(torch.bfloat16).cuda().repeat(8, 1, 1)
    Kt = torch.randn(8, 128, 2048, generator=g).to(torch.bfloat16).cuda().repeat(8, 1, 1)
    S = torch.empty((64, 2048, 2048), dtype=torch.bfloat16, device="cuda")
    t = timeit(lambda: h.matmul(Q, Kt, out=S, alpha=128 ** -0.5))
    gbs = 603979776 / t / 1e9
    out["batched_64x2048x2048x128_bf16"] = {"GB/s": gbs, "TFLOP/s": 6.872e10 / t / 1e12,
                                            "frac_of_measured_hbm": gbs / peaks["hbm_gbs"],
                                            "ms": t * 1e3, "kernel": h.last_kernel}
    # write-dominated (512 MiB out of 576 MiB): a plain fill of the output and the vendor
    # library's batched matmul on the same buffers, for context only
    t_fill = timeit(lambda: S.zero_())
    out["batched_64x2048x2048x128_bf16"]["fill_of_the_output_GB/s"] = S.numel() * 2 / t_fill / 1e9
    t_lib = timeit(lambda: torch.bmm(Q, Kt, out=S))
    out["batched_64x2048x2048x128_bf16"]["library_torch_bmm_GB/s"] = 603979776 / t_lib / 1e9
    del Q, Kt, S
    # fp16 1024^3 with column-major B: launch-latency scale, absolute time only
    A1 = (torch.rand(1024, 1024, generator=g) * 2 - 1).to(torch.float16).cuda()
    B1 = (torch.rand(1024, 1024, generator=g) * 2 - 1).to(torch.float16).cuda().t()
    C1 = torch.empty((1024, 1024), dtype=torch.float16, device="cuda")
    t = timeit(lambda: h.matmul(A1, B1, out=C1), iters=20, flush_l2=True)
    out["fp16_1024^3_colmajorB"] = {"us": t * 1e6, "TFLOP/s": 2.147e9 / t / 1e12,
                                    "kernel": h.last_kernel}
    h.check()
    return out


def run_ours(args):
    import torch
    import torch.distributed as dist

    import __graft_entry__ as entry
    pkg = entry.load_package()

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        # NCCL prints its version banner on stdout; the JSON line must be alone there
        os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    else:
        torch.cuda.set_device(0)
        local = 0
    peaks = load_peaks()
    h = pkg.Handle(local)
    if args.path:
        h.set_matmul_path(args.path)

    c0, c1 = pkg.shard_range(N, world, rank, 256)
    A, Bs, bias = make_inputs(torch, c0, c1)
    A_pin, B_pin, bias_pin = A.pin_memory(), Bs.pin_memory(), bias.pin_memory()
    Ad, Bd, bd = A_pin.cuda(non_blocking=True), B_pin.cuda(non_blocking=True), bias_pin.cuda(non_blocking=True)
    Cd = torch.empty((M, c1 - c0), dtype=torch.bfloat16, device="cuda")
    torch.cuda.synchronize()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def step():
        h.matmul(Ad, Bd, out=Cd, bias=bd)

    for _ in range(max(3, args.warmup)):
        step()
    h.check()
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    launches0 = h.launch_count
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_begin = time.perf_counter()
    ev0.record()
    for _ in range(args.steps):
        step()
    ev1.record()
    ev1.synchronize()
    t_end = time.perf_counter()
    barrier()
    clocks = sampler.stop(t_begin, t_end) if rank == 0 else None
    launches = h.launch_count - launches0
    h.check()
    elapsed = ev0.elapsed_time(ev1) * 1e-3
    if world > 1:
        t = torch.tensor([elapsed], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        elapsed = float(t.item())
    sec_per_step = elapsed / args.steps
    value = FLOPS / sec_per_step / 1e12

    # The SM clock INSIDE the kernel under the same load (NVML's samples are too
    # slow for a 15 ms region): the same burst again, untimed, with the kernel's own
    # probe on (cycles and nanoseconds of the first CTA's MMA warp, last launch).
    if rank == 0 and clocks is not None:
        try:
            h.set_matmul_path("auto:d128")
            for _ in range(args.steps):
                step()
            cyc, ns = h.probe_clock()
            if ns:
                mhz = cyc / ns * 1e3
                clocks["sm_mhz_in_kernel"] = round(mhz, 1)
                clocks["tensor_peak_at_that_clock_tflops"] = round(2250.0 * mhz / 1965.0, 1)
        finally:
            h.set_matmul_path("auto")

    # ---- end to end through the host-buffer C-ABI call (pinned host memory in,
    # pinned host memory out, copies inside the timed region)
    C_pin = torch.empty((M, c1 - c0), dtype=torch.bfloat16).pin_memory()
    h.matmul_host(A_pin, B_pin, C_pin, bias=bias_pin)
    e2e_steps = max(2, min(args.steps, 5))
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        h.matmul_host(A_pin, B_pin, C_pin, bias=bias_pin)
    torch.cuda.synchronize()
    e2e_t = (time.perf_counter() - t0) / e2e_steps
    if world > 1:
        t = torch.tensor([e2e_t], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_t = float(t.item())
    h2d = A_pin.numel() * 2 + B_pin.numel() * 2 + bias_pin.numel() * 2
    d2h = C_pin.numel() * 2
    e2e = {"value": FLOPS / e2e_t / 1e12, "unit": UNIT, "h2d_bytes_per_step": h2d,
           "d2h_bytes_per_step": d2h, "ms_per_step": e2e_t * 1e3}
    assert torch.equal(C_pin, Cd.cpu()), "host-buffer call and device call disagree"

    # ---- N > 1: the same step with the full output assembled on every rank
    gather = None
    if world > 1:
        gather = {"bytes_received_per_gpu": int(M * (N - (c1 - c0)) * 2)}
        spans = pkg.dist.column_shards(N, world, 256)

        def timed(fn, iters):
            for _ in range(2):
                fn()
            barrier()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(iters):
                fn()
            b.record()
            b.synchronize()
            barrier()
            t = torch.tensor([a.elapsed_time(b) * 1e-3 / iters], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return float(t.item())

        iters = max(2, min(args.steps, 10))
        try:
            full = torch.empty((M, N), dtype=torch.bfloat16, device="cuda")

            def nccl_step():
                h.matmul(Ad, Bd, out=Cd, bias=bd)
                pkg.dist.all_gather_columns(Cd, spans, out=full)
            tn = timed(nccl_step, iters)
            gather["nccl_all_gather"] = {"value": FLOPS / tn / 1e12, "unit": UNIT, "ms_per_step": tn * 1e3}
            del full
        except Exception as ex:  # report, keep the main number
            gather["nccl_all_gather"] = {"error": repr(ex)[:200]}
        try:
            pg = pkg.dist.PushGather(M, N, torch.bfloat16, torch.device("cuda", local))

            def push_step():
                pg.matmul(h, Ad, Bd, c0, bias_shard=bd)
                pg.wait()
            tp = timed(push_step, iters)
            h.check()
            ok = bool(torch.equal(pg.full[:, c0:c1], Cd))
            gather["fused_push"] = {"value": FLOPS / tp / 1e12, "unit": UNIT, "ms_per_step": tp * 1e3,
                                    "matches_local_shard": ok}
        except Exception as ex:
            gather["fused_push"] = {"error": repr(ex)[:200]}

    line = None
    if rank == 0:
        long_run = elapsed > 1.0
        peak = peaks["bf16_sustained"] if long_run else peaks["bf16_burst"]
        per_gpu = value / world
        roofline = {"bound": "tensor", "achieved": per_gpu, "peak": peak, "unit": UNIT,
                    "frac": per_gpu / peak,
                    "peak_kind": ("sustained" if long_run else "burst") + " cuBLAS bf16, " +
                                 peaks["source"],
                    "frac_of_nominal_2250": per_gpu / 2250.0,
                    "traffic": NCU_TRAFFIC_BYTES, "algorithmic_bytes": ALG_BYTES,
                    "kernel": h.last_kernel}
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": sec_per_step * 1e3,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "bf16 GEMM M=N=K=8192 row-major A/B, fp32 accumulate, bf16 out, "
                                   "fused per-column bias", "seed": SEED,
                       "sharding": f"columns of B and C over {world} rank(s), no collective",
                       "l2": "A+B+C = 384 MiB per step, larger than the 126 MB L2"},
            "e2e": e2e, "gpu_launches": int(launches), "clocks": clocks, "roofline": roofline,
        }
        if gather is not None:
            line["gather"] = gather

    # ---- CPU baseline: the checker's fp32-accumulate port on a bounded row sample
    if rank == 0 and world == 1:
        import numpy as np

        import oracle as ko
        ko.build()
        bits = lambda t: t.view(torch.int16).numpy().view(np.uint16)
        Ab, Bb, bb = bits(A), bits(Bs), bits(bias)
        cpu_step(ko, Ab, Bb, bb, 32)
        t0 = time.perf_counter()
        got = cpu_step(ko, Ab, Bb, bb, CPU_SAMPLE_ROWS)
        dt = time.perf_counter() - t0
        cores = ko.num_threads()
        line["cpu_baseline"] = {
            "value": 2.0 * CPU_SAMPLE_ROWS * N * K / dt / 1e12, "unit": UNIT, "cores": cores,
            "kind": "port",
            "sample": f"rows [0,{CPU_SAMPLE_ROWS}) of the output (all of B and K), "
                      f"{dt:.1f} s on {cores} OpenMP threads"}
        # the CPU sample doubles as a parity spot check of the timed output
        dev = Cd[:CPU_SAMPLE_ROWS].float().cpu()
        cpu = torch.from_numpy(got[:CPU_SAMPLE_ROWS].view(np.int16)).view(torch.bfloat16).float()
        line["cpu_baseline"]["max_abs_diff_vs_gpu"] = float((dev - cpu).abs().max())
        if not args.no_extra:
            del Ad, Bd, Cd
            torch.cuda.empty_cache()
            line["extra"] = secondary(torch, pkg, h, peaks)

    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if rank == 0:
        print(json.dumps(line))


def run_profile_case(args):
    """Launches one kernel family a few times on a small case (inputs larger than
    L2, a few hundred MB on the device) so that a profiler capture ends quickly.
    Prints nothing that counts as a benchmark value."""
    import torch

    import __graft_entry__ as entry
    pkg = entry.load_package()
    abi = pkg.abi
    torch.cuda.set_device(0)
    h = pkg.Handle(0)
    if args.path:
        h.set_matmul_path(args.path)
    g = torch.Generator(device="cpu").manual_seed(1)
    case = args.profile_case
    if case == "gemm":
        m, n, k = 8192, 8192, 4096   # same tile grid as the benchmark, half of its K loop
        A = (torch.randn(m, k, generator=g) * k ** -0.5).to(torch.bfloat16).cuda()
        B = (torch.randn(k, n, generator=g) * k ** -0.5).to(torch.bfloat16).cuda()
        bias = torch.zeros(n, dtype=torch.bfloat16, device="cuda")
        C = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
        fn = lambda: h.matmul(A, B, out=C, bias=bias)
    elif case == "gelu":
        x = torch.randn(1, 1 << 27, generator=g).to(torch.bfloat16).cuda()
        y = torch.empty_like(x)
        prog = pkg.programs.affine_gelu_tanh(abi.BF16, 0.5, 0.1)
        fn = lambda: h.elementwise(prog, [x], y)
    elif case == "rowsum":
        X = torch.randn(32768, 4096, generator=g).to(torch.bfloat16).cuda()
        s = torch.empty((32768, 1), dtype=torch.float32, device="cuda")
        fn = lambda: h.reduce(X, axis=1, out=s)
    elif case == "decode":
        X = torch.randn(16, 8192, generator=g).to(torch.bfloat16).cuda()
        W = (torch.randn(8192, 14336, generator=g) * 0.02).to(torch.bfloat16).cuda()
        o = torch.empty((16, 14336), dtype=torch.bfloat16, device="cuda")
        fn = lambda: h.matmul(X, W, out=o)
    elif case == "batched":
        Q = torch.randn(32, 2048, 128, generator=g).to(torch.bfloat16).cuda()
        Kt = torch.randn(32, 128, 2048, generator=g).to(torch.bfloat16).cuda()
        S = torch.empty((32, 2048, 2048), dtype=torch.bfloat16, device="cuda")
        fn = lambda: h.matmul(Q, Kt, out=S, alpha=128 ** -0.5)
    else:
        raise SystemExit(f"unknown profile case {case}")
    for _ in range(6):
        fn()
    h.check()
    print(json.dumps({"profile_case": case, "kernel": h.last_kernel, "launches": h.launch_count}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--path", default="", help="force a matmul kernel family (tests/profiling)")
    ap.add_argument("--no-extra", action="store_true", help="skip the secondary configurations")
    ap.add_argument("--profile-case", default="",
                    help="gemm|gelu|rowsum|decode|batched: a small case for a profiler capture")
    args = ap.parse_args()
    if args.profile_case:
        run_profile_case(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
