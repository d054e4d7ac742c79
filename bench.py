#!/usr/bin/env python
"""Benchmark of the hot path:  python bench.py --gpus N --steps K --warmup W [--impl reference]

One "step" is one pass of the hot path over one resident batch: the bf16 GEMM
C[m,n] = A[m,k] B[n,k]^T at m=n=k=8192 (the shape the headline metric is quoted on).
At N > 1 (launched by torchrun, one process per GPU) every rank holds A and its own
8192-column block of B and computes its own column block of C — the column-sharded
layout, weak scaling, no data-path collective.

Prints ONE JSON line (rank 0):
  value      whole-job TFLOP/s, inputs resident in HBM, CUDA-event timed, max over ranks
  e2e        the same metric through the torch operator with HOST buffers: pinned-host -> device
             copies of A and B and the device -> host copy of C inside the timed region
  roofline   the GEMM kernel against the measured cuBLAS bf16 peak (MEASURED_PEAKS.json)
  cpu_baseline  the oracle's CPU form (torch fp32 matmul on the host cores) on a bounded row band
  plus comparators measured in the same process: cuBLAS (torch.matmul), the reference project's
  own mma.sync kernel compiled for sm_100a (oracle/_ref, if built), and the RMSNorm kernels' GB/s.

--impl reference times the reference path's CPU form (the reference has no CPU code of its
own; its formula restated as torch fp32 matmul) on the host cores, rank 0 only.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import threading
import time

REPO = os.path.dirname(os.path.abspath(__file__))
if REPO not in sys.path:
    sys.path.insert(0, REPO)

M = N = K = 8192
WORKLOAD = "bf16 GEMM m=n=k=8192 TN (A[m,k] row-major, B[n,k]), U[-1,1] seed 1 (benchmark configs[1])"
METRIC = "hgemm_bf16_tflops_8192"
UNIT = "TFLOP/s"


def bench_config(world: int) -> dict:
    """The `config` object of the JSON line; both arms (ours, --impl reference) print the same one."""
    w = WORKLOAD if world == 1 else WORKLOAD + (f"; x{world} ranks, rank r owns column block r of "
                                                f"B[{N * world},{K}] (A replicated), no gather")
    return {"workload": w, "l2": f"inputs+output {2 * (M * K + N * K + M * N) / 1e6:.0f} MB per step vs 126 MB L2: "
                                 "larger than L2, no flush between iterations"}


def measured_peaks() -> dict:
    path = os.path.join(REPO, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        d["_source"] = "measured"
        return d
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "_source": "fallback"}


def ncu_traffic(kernel_key: str):
    """Per-launch DRAM bytes of a kernel from the committed ncu summary (profiles/traffic.json), or None."""
    path = os.path.join(REPO, "profiles", "traffic.json")
    if not os.path.exists(path):
        return None
    with open(path) as f:
        return json.load(f).get(kernel_key)


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons of one GPU while the timed region runs."""

    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.rows = []
        self.proc = None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-i", str(self.index),
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 7:
                self.rows.append(parts)

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
            self.thread.join(timeout=2)

    def summary(self) -> dict:
        sm, mx, reasons = [], [], set()
        for r in self.rows:
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def use_all_host_threads() -> int:
    """torchrun exports OMP_NUM_THREADS=1; the CPU legs are meant to use every core this process may run on."""
    import torch

    n = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    torch.set_num_threads(max(1, n))
    return torch.get_num_threads()


def cpu_gemm_baseline(target_seconds: float = 12.0) -> dict:
    """torch CPU fp32 matmul on a row band of the 8192^3 problem (A band [rows, k] x full B)."""
    import torch

    use_all_host_threads()
    torch.manual_seed(1)
    b = (torch.rand(N, K) * 2 - 1).to(torch.bfloat16).float()
    rows = 256
    a = (torch.rand(rows, K) * 2 - 1).to(torch.bfloat16)
    t0 = time.perf_counter()
    torch.nn.functional.linear(a.float(), b)
    dt = time.perf_counter() - t0
    # grow the band towards the time target, bounded by the full problem
    rows2 = int(min(M, max(rows, rows * target_seconds / max(dt, 1e-3) / 3)))
    rows2 = max(256, rows2 // 256 * 256)
    a = (torch.rand(rows2, K) * 2 - 1).to(torch.bfloat16)
    best = None
    for _ in range(3):
        t0 = time.perf_counter()
        torch.nn.functional.linear(a.float(), b)
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    tflops = 2.0 * rows2 * N * K / best / 1e12
    return {"value": tflops, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"torch CPU fp32 F.linear on a {rows2}-row band of A against all of B[{N},{K}] "
                      f"(best of 3, {best * 1e3:.1f} ms; widening B to fp32 not timed)",
            "host_cpus": os.cpu_count()}


def run_reference_arm(args) -> None:
    """The reference path's CPU form on the host cores; rank 0 only."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import torch

    use_all_host_threads()
    torch.manual_seed(1)
    b = (torch.rand(N, K) * 2 - 1).to(torch.bfloat16).float()
    rows = 1024
    a = (torch.rand(rows, K) * 2 - 1).to(torch.bfloat16)
    for _ in range(max(args.warmup, 1)):
        torch.nn.functional.linear(a.float(), b)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        torch.nn.functional.linear(a.float(), b)
    dt = time.perf_counter() - t0
    tflops = 2.0 * rows * N * K * args.steps / dt / 1e12
    cb = {"value": tflops, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
          "sample": f"each step = torch CPU fp32 F.linear of a {rows}-row band of A against all of B[{N},{K}]"}
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": tflops, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": bench_config(int(os.environ.get("WORLD_SIZE", "1"))),
        "note": "the reference has no CPU implementation; this is its oracle formula (src/impl/sgemm_impl.h:17-25) "
                "as an fp32 CPU matmul on a bounded row band",
        "cpu_baseline": cb,
        "e2e": {"value": tflops, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def time_cuda(fn, steps: int, warmup: int):
    """ms per call: CUDA events on the current stream around `steps` back-to-back calls."""
    import torch

    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps


def rmsnorm_numbers(peaks: dict, steps: int, warmup: int, rows: int = 32768) -> dict:
    """RMSNorm fwd/bwd achieved GB/s at [32768, H] bf16 (algorithmic bytes 4RH+4H and 6RH+8H)."""
    import torch

    from peakgemm_b200 import capi

    out = {}
    R = rows
    for H in (4096, 8192):
        g = torch.Generator(device="cuda").manual_seed(3)
        x = torch.randn(R, H, device="cuda", generator=g).to(torch.bfloat16)
        dy = torch.randn(R, H, device="cuda", generator=g).to(torch.bfloat16)
        gamma = (1 + 0.1 * torch.randn(H, device="cuda", generator=g)).float()
        y, dx, dg = torch.empty_like(x), torch.empty_like(x), torch.empty_like(gamma)
        ws = torch.empty(capi.rmsnorm_bwd_workspace_bytes(R, H) // 4, device="cuda")
        # x (+dy) and the outputs are 0.5-1.6 GB per call: far larger than the 126 MB L2
        t_f = time_cuda(lambda: capi.rmsnorm_fwd(y, x, gamma), steps, warmup)
        t_b = time_cuda(lambda: capi.rmsnorm_bwd(dx, dg, dy, x, gamma, ws), steps, warmup)
        bf, bb = 4 * R * H + 4 * H, 6 * R * H + 8 * H
        out[f"h{H}"] = {
            "fwd_ms": t_f, "fwd_gbs": bf / t_f / 1e6, "fwd_frac_of_measured_hbm": bf / t_f / 1e6 / peaks["hbm_gbs"],
            "bwd_ms": t_b, "bwd_gbs": bb / t_b / 1e6, "bwd_frac_of_measured_hbm": bb / t_b / 1e6 / peaks["hbm_gbs"],
        }
        del x, dy, y, dx
    return out


def probes() -> dict:
    """What this GPU allows with nothing in the way (pg_probe_*): back-to-back tcgen05.mma on resident tiles, and a
    streaming copy.  The reference's counterparts are test/cpp/test_wmma_compute.cpp and test_memory_bandwidth.cpp."""
    import torch

    from peakgemm_b200 import capi

    out = {}
    for name, is_bf16 in (("bf16", True), ("fp16", False)):
        burst, ms_b = capi.probe_tensor_peak(is_bf16, 2000)          # ~0.7 ms: the length of one 8192^3 GEMM
        sustained, ms_s = capi.probe_tensor_peak(is_bf16, 60000)     # ~25 ms under the power cap
        out[f"mma_{name}_tflops_burst"] = burst
        out[f"mma_{name}_tflops_sustained"] = sustained
    src = torch.empty(512 << 20, dtype=torch.uint8, device="cuda")
    dst = torch.empty_like(src)
    t = time_cuda(lambda: capi.probe_copy(dst, src), 20, 3)
    out["copy_gbs"] = 2 * src.numel() / t / 1e6
    out["what"] = "tcgen05.mma.cta_group::2 256x256x16 issued back to back on all SM pairs, pseudo-random operands " \
                  "resident in shared memory, no loads; 128-bit streaming copy of 512 MiB"
    return out


def shape_sweep(peaks: dict) -> list:
    """benchmark configs 2 and 3: every shape, ours (automatic configuration) against cuBLAS on the same GPU.

    Throughput timing as the reference's Python benchmark does it (test/test_gemm.py:62-96): several
    independent (B, C) sets are rotated through back-to-back launches, enough of them (>= 256 MB of B) that a
    weight matrix is never found in the 126 MB L2 from its previous use; CUDA events around the whole loop; ours and
    cuBLAS in alternating rounds, medians of 4.
    Roofline time = max(2mnk / measured bf16 peak, 2(mk+nk+mn) / measured HBM peak)."""
    import torch

    from peakgemm_b200 import capi

    shapes = [("config2", s, s, s, dt) for s in (2048, 4096, 8192, 16384) for dt in (torch.float16, torch.bfloat16)]
    shapes += [("config3", m, n, k, torch.bfloat16) for m in (16, 128, 1024, 4096)
               for (n, k) in ((4096, 4096), (14336, 4096), (4096, 14336), (128256, 4096))]
    # the sharded benchmark shape (configs[4]): one of 8 ranks' blocks, a quarter of the problem, the whole problem
    shapes += [("config5", 32768, 4096, 16384, torch.bfloat16), ("config5", 8192, 32768, 16384, torch.bfloat16),
               ("config5", 32768, 32768, 16384, torch.bfloat16)]
    rows = []
    g = torch.Generator(device="cuda").manual_seed(2)
    for tag, m, n, k, dt in shapes:
        nbuf = max(1, min(16, -(-(256 << 20) // (2 * n * k))))
        if tag in ("config2", "config5"):
            a = (torch.rand(m, k, device="cuda", generator=g) * 2 - 1).to(dt)
            bs = [(torch.rand(n, k, device="cuda", generator=g) * 2 - 1).to(dt) for _ in range(nbuf)]
        else:
            a = torch.randn(m, k, device="cuda", generator=g).to(dt)
            bs = [(0.02 * torch.randn(n, k, device="cuda", generator=g)).to(dt) for _ in range(nbuf)]
        cs = [torch.empty(m, n, dtype=dt, device="cuda") for _ in range(nbuf)]
        iters = max(nbuf, 32 if m * n * k < 2 ** 38 else 8)

        def loop(fn):
            for i in range(min(iters, 4)):
                fn(i % nbuf)
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for i in range(iters):
                fn(i % nbuf)
            e1.record()
            torch.cuda.synchronize()
            return e0.elapsed_time(e1) / iters

        need = capi.hgemm_workspace_bytes(m, n, k)       # > 0: the last partial wave is split over k (what the
        ws = torch.empty(need, dtype=torch.uint8, device="cuda") if need else None     # torch operator does too)
        # the two libraries take turns (4 rounds, the order alternating) and the medians are compared: both sit on
        # the same power cap, and whichever runs second on a warm GPU would otherwise look slower
        runs_o, runs_c = [], []
        for r in range(4):
            for which in ((0, 1) if r % 2 == 0 else (1, 0)):
                if which == 0:
                    runs_o.append(loop(lambda i: capi.hgemm_ws(cs[i], a, bs[i], ws)))
                else:
                    runs_c.append(loop(lambda i: torch.matmul(a, bs[i].t(), out=cs[i])))
        t_o, t_c = statistics.median(runs_o), statistics.median(runs_c)
        fl, by = 2.0 * m * n * k, 2.0 * (m * k + n * k + m * n)
        t_roof = max(fl / (peaks["bf16_tflops"] * 1e12), by / (peaks["hbm_gbs"] * 1e9)) * 1e3
        rows.append({"config": tag, "dtype": str(dt)[6:], "m": m, "n": n, "k": k, "weight_sets": nbuf,
                     "ours_us": t_o * 1e3, "cublas_us": t_c * 1e3, "ours_tflops": fl / t_o / 1e9,
                     "ours_gbs": by / t_o / 1e6, "roofline_us": t_roof * 1e3, "frac_of_roofline": t_roof / t_o,
                     "speed_vs_cublas": t_c / t_o, "tail_split_workspace_bytes": need,
                     "persistent_config": list(capi.hgemm_config(m, n, k)) if m > 128 else None})
        del a, bs, cs
    assert capi.device_status() == 0
    return rows


def chain_sweep() -> list:
    """RMSNorm -> projection at the LLM shapes of benchmark config 3 (k = 4096 hidden size), four ways on one GPU:
      two_op      rms_norm_fwd then gemm_peak (y written and re-read)
      fused       rms_norm_rstd then gemm_peak_fused over the raw x (rstd applied in the epilogue)
      fused_pdl   the same with the GEMM launched under programmatic stream serialisation (main loop overlaps
                  the rstd kernel, only the epilogue waits)
      torch       torch.nn.functional.rms_norm + F.linear (cuBLAS), the library comparator
    plus the GEMM, the norm and the rstd kernel alone.  Weight sets are rotated so that no weight is found in L2
    from its previous use.  Each case is timed twice: 32 chains captured in one CUDA graph and replayed (device
    time) and launched eagerly from Python (adds the host cost of two operator calls per chain)."""
    import torch
    import torch.nn.functional as F

    import peakgemm_b200 as pg

    rows = []
    g = torch.Generator(device="cuda").manual_seed(5)
    k = 4096
    for m in (16, 128, 1024, 4096):
        for n in (4096, 14336):
            nbuf = max(2, min(16, -(-(256 << 20) // (2 * n * k))))
            x = torch.randn(m, k, device="cuda", generator=g).to(torch.bfloat16)
            gamma = (1 + 0.1 * torch.randn(k, device="cuda", generator=g)).float()
            gamma16 = gamma.to(torch.bfloat16)
            ws = [(0.02 * torch.randn(n, k, device="cuda", generator=g)).to(torch.bfloat16) for _ in range(nbuf)]
            wfs = [pg.fold_gamma(w, gamma) for w in ws]
            outs = [torch.empty(m, n, dtype=torch.bfloat16, device="cuda") for _ in range(nbuf)]
            y = torch.empty_like(x)
            rstd = torch.empty(m, device="cuda")
            iters = 32

            def loop(fn):
                """(graph, eager) us per chain: `iters` chains captured in one CUDA graph and replayed (device
                time, no host launch cost), and the same chains launched eagerly from Python."""
                for i in range(4):
                    fn(i % nbuf)
                torch.cuda.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for i in range(iters):
                    fn(i % nbuf)
                e1.record()
                torch.cuda.synchronize()
                eager = e0.elapsed_time(e1) / iters * 1e3
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph):
                    for i in range(iters):
                        fn(i % nbuf)
                best = float("inf")
                for _ in range(4):                    # the first replay is the warm-up
                    e0.record()
                    graph.replay()
                    e1.record()
                    torch.cuda.synchronize()
                    best = min(best, e0.elapsed_time(e1) / iters * 1e3)
                return best, eager

            def two_op(i):
                pg.rms_norm_fwd(y, x, gamma)
                pg.gemm_peak(outs[i], y, ws[i])

            def torch_chain(i):
                torch.matmul(F.rms_norm(x, (k,), gamma16, 1e-6), ws[i].t(), out=outs[i])

            cases = {
                "two_op": two_op,
                "fused": lambda i: pg.rms_norm_linear(outs[i], x, wfs[i], rstd=rstd, pdl=False),
                "fused_pdl": lambda i: pg.rms_norm_linear(outs[i], x, wfs[i], rstd=rstd, pdl=True),
                "gemm_only": lambda i: pg.gemm_peak(outs[i], x, ws[i]),
                "norm_only": lambda i: pg.rms_norm_fwd(y, x, gamma),
                "rstd_only": lambda i: torch.ops.PeakGemm.rms_norm_rstd(rstd, x, 1e-6),
                "torch": torch_chain,
            }
            t = {}
            for name, fn in cases.items():
                t[f"{name}_us"], t[f"{name}_eager_us"] = loop(fn)
            rows.append({"m": m, "n": n, "k": k, "weight_sets": nbuf, **t})
            del ws, wfs, outs
    return rows


def e2e_ms(a, b, c, steps: int):
    """ms per step of PeakGemm.gemm_peak with HOST buffers: every step copies ITS inputs host -> device from pinned
    memory, runs the operator and reads ITS result back.  Three buffer sets and three streams (copy-in, operator,
    copy-out) let step i+1's upload and step i-1's download overlap step i's GEMM: PCIe is full duplex, the link is
    the bottleneck, not the kernel."""
    import torch

    import PeakGemm

    ah, bh = a.cpu().pin_memory(), b.cpu().pin_memory()
    ch = torch.empty(c.shape, dtype=c.dtype).pin_memory()
    nb = 3
    ad = [torch.empty_like(a) for _ in range(nb)]
    bd = [torch.empty_like(b) for _ in range(nb)]
    cd = [torch.empty_like(c) for _ in range(nb)]
    s_in, s_op, s_out = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()
    ev_in = [torch.cuda.Event() for _ in range(nb)]
    ev_op = [torch.cuda.Event() for _ in range(nb)]
    ev_out = [torch.cuda.Event() for _ in range(nb)]

    def run(n_steps):
        main = torch.cuda.current_stream()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        t0.record(main)
        for st in (s_in, s_op, s_out):
            st.wait_event(t0)
        for s_ in range(n_steps):
            i = s_ % nb
            with torch.cuda.stream(s_in):
                if s_ >= nb:
                    s_in.wait_event(ev_op[i])          # the GEMM that read this buffer set has finished
                ad[i].copy_(ah, non_blocking=True)
                bd[i].copy_(bh, non_blocking=True)
                ev_in[i].record(s_in)
            with torch.cuda.stream(s_op):
                s_op.wait_event(ev_in[i])
                if s_ >= nb:
                    s_op.wait_event(ev_out[i])         # the previous result in this set has been read back
                PeakGemm.gemm_peak(cd[i], ad[i], bd[i])
                ev_op[i].record(s_op)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_op[i])
                ch.copy_(cd[i], non_blocking=True)
                ev_out[i].record(s_out)
        for st in (s_in, s_op, s_out):
            main.wait_stream(st)
        t1.record(main)
        torch.cuda.synchronize()
        return t0.elapsed_time(t1) / n_steps

    e2e_steps = max(6, min(steps, 12))
    run(3)
    return run(e2e_steps), e2e_steps


def reference_style_timing(a, b, c, flops: float) -> dict:
    """The two ways the reference times its kernel, applied to ours on the same inputs:
    a single launch between two events right after a device synchronisation, nothing warm beyond the module itself
    (test/cpp/test_gemm_half.cpp:109-129; median and best of 5 such launches, an L2 flush before each), and the
    average self-CUDA time torch.profiler attributes to the kernel over 40 calls after 10 warm-ups
    (test/test_gemm.py:69-96)."""
    import torch

    from peakgemm_b200 import capi

    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    cold = []
    for _ in range(5):
        flush.zero_()                       # 256 MB written: nothing of A, B or C is left in the 126 MB L2
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        capi.hgemm(c, a, b)
        e1.record()
        torch.cuda.synchronize()
        cold.append(e0.elapsed_time(e1))
    out = {"single_cold_launch_ms_median": statistics.median(cold), "single_cold_launch_ms_best": min(cold),
           "single_cold_launch_tflops_median": flops / (statistics.median(cold) * 1e-3) / 1e12}
    try:
        from torch.profiler import ProfilerActivity, profile

        for _ in range(10):
            capi.hgemm(c, a, b)
        torch.cuda.synchronize()
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            for _ in range(40):
                capi.hgemm(c, a, b)
            torch.cuda.synchronize()
        rows = [e for e in prof.key_averages() if "hgemm" in e.key]
        if rows:
            us = max(rows, key=lambda e: e.self_device_time_total).self_device_time_total / 40.0
            out["profiler_self_cuda_ms_avg_of_40"] = us / 1e3
            out["profiler_tflops"] = flops / (us * 1e-6) / 1e12
            out["profiler_note"] = ("back-to-back launches overlap (programmatic dependent launch): a kernel's interval "
                                    "as the profiler records it includes its wait for the previous one, so the sum of "
                                    "the intervals exceeds the elapsed time")
    except Exception as exc:  # noqa: BLE001  (the profiler needs CUPTI; report rather than fail the bench)
        out["profiler_unavailable"] = repr(exc)[:200]
    return out


def config5_block(world: int, rank: int, steps: int = 3) -> dict:
    """benchmark config 5 on the ranks of this run, as part of the default JSON line: m = n = 32768, k = 16384 bf16,
    B column-sharded over the ranks with A replicated (STRONG scaling: the problem is fixed, N = 1 is the
    denominator).  Timed without a gather, with the NCCL all-gather (native shard-major result, and copied to
    row-major), with the gather fused into the GEMM epilogue as peer stores (row-major on every rank) and as stores that
    the NVLink switch replicates (multicast).  CUDA events,
    max over ranks.  `parity`: 16 sampled rows of this rank's block against an fp32 product of the same inputs
    (acceptance bound), and at N > 1 the fused result against the NCCL result bit for bit."""
    import math

    import torch
    import torch.distributed as dist

    from peakgemm_b200 import capi
    from peakgemm_b200.dist import PeerMatrix, ShardedGemm

    m = n = 32768
    k = 16384
    sg = ShardedGemm(n)
    g = torch.Generator(device="cuda").manual_seed(4)
    a = (torch.rand(m, k, device="cuda", generator=g) * 2 - 1).to(torch.bfloat16)
    g.manual_seed(400 + rank)
    b = (torch.rand(sg.n_local, k, device="cuda", generator=g) * 2 - 1).to(torch.bfloat16)
    out = torch.empty(m, sg.n_local, dtype=torch.bfloat16, device="cuda")

    def timed(fn, reps):
        for _ in range(2):
            fn()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / reps], device="cuda")
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.item()

    flop = 2.0 * m * n * k
    res = {"workload": "bf16 GEMM m=n=32768 k=16384, B column-sharded over the ranks, A replicated (benchmark "
                       "configs[4]); strong scaling", "n_gpus": world, "steps": steps, "flop": flop}
    res["no_gather_ms"] = timed(lambda: sg.local(a, b, out=out), steps)
    res["tflops"] = flop / (res["no_gather_ms"] * 1e-3) / 1e12
    # parity of this rank's block on sampled rows
    rows = (torch.arange(16, device="cuda") * (m // 16) + 5)
    ref = a[rows].float() @ b.float().t()
    tol = (2e-2 * math.sqrt(k / 4096.0) + 2.0 ** -8) * ref.abs().max().item()
    ok = torch.tensor([int((out[rows].float() - ref).abs().max().item() <= tol)], device="cuda")
    del ref
    if world == 1:
        full_b = b
        t_cublas = timed(lambda: torch.matmul(a, full_b.t(), out=out), steps)
        res["cublas_ms"] = t_cublas
        res["cublas_tflops"] = flop / (t_cublas * 1e-3) / 1e12
    else:
        res["nccl_gather_shard_major_ms"] = timed(
            lambda: sg.gathered(a, b, layout="shard_major", bands=4, max_sms=140), steps)
        res["nccl_gather_ms"] = timed(lambda: sg.gathered(a, b, layout="row_major", bands=4, max_sms=140), steps)
        nccl = sg.gathered(a, b, layout="row_major", bands=4, max_sms=140)
        pm = PeerMatrix(m, n, torch.bfloat16)
        res["fused_gather_ms"] = timed(lambda: sg.gathered_fused(pm, a, b), steps)
        fused = sg.gathered_fused(pm, a, b)
        torch.cuda.synchronize()
        same = torch.equal(fused, nccl)
        ok = ok * int(same)
        del fused
        pm.close()
        # the gather done by the NVLink switch (multimem.st through a multicast mapping), where the machine has one
        from peakgemm_b200.dist import MulticastMatrix

        try:
            mm = MulticastMatrix(m, n, torch.bfloat16)
        except RuntimeError as exc:              # raised on every rank or on none (the constructor agrees first)
            mm = None
            res["multicast_unavailable"] = str(exc)[:200]
        if mm is not None:
            res["multicast_gather_ms"] = timed(lambda: sg.gathered_multicast(mm, a, b), steps)
            mc = sg.gathered_multicast(mm, a, b)
            torch.cuda.synchronize()
            dist.barrier()
            ok = ok * int(torch.equal(mc, nccl))
            del mc
            mm.close()
        else:
            res["multicast_gather_ms"] = None
        del nccl
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        res["gather_bytes_received_per_gpu"] = 2 * m * (n - sg.n_local)
    res["parity"] = bool(ok.item())
    res["device_status"] = capi.device_status()
    del a, b, out
    torch.cuda.empty_cache()
    return res


def rmsnorm_sharded_block(world: int, rank: int, peaks: dict, steps: int = 30) -> dict:
    """benchmark config 4 ([32768, H] bf16, H = 4096 and 8192) with the rows sharded over the ranks of this run
    (strong scaling): forward, backward with the local dgamma only, and backward with the global dgamma
    (all-gather of the partial vectors, summed in rank order).  Aggregate GB/s = algorithmic bytes of the WHOLE
    problem (4RH + 4H, 6RH + 8H) / max-over-ranks time."""
    import torch
    import torch.distributed as dist

    from peakgemm_b200.dist import ShardedRmsNorm

    R = 32768
    out = {"n_gpus": world, "rows_total": R}
    for H in (4096, 8192):
        sn = ShardedRmsNorm(R)
        g = torch.Generator(device="cuda").manual_seed(3 + 10 * rank)
        x = torch.randn(sn.rows_local, H, device="cuda", generator=g).to(torch.bfloat16)
        dy = torch.randn(sn.rows_local, H, device="cuda", generator=g).to(torch.bfloat16)
        gamma = (1 + 0.1 * torch.randn(H, device="cuda", generator=torch.Generator(device="cuda").manual_seed(3))).float()
        y = torch.empty_like(x)

        def timed(fn):
            # the block runs right after 24 ms GEMMs at the power cap: a pause, then warm-up launches that flow
            # straight into the timed ones (no idle gap in front of the first timed launch)
            torch.cuda.synchronize()
            if world > 1:
                dist.barrier()
            time.sleep(0.2)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            for _ in range(5):
                fn()
            e0.record()
            for _ in range(steps):
                fn()
            e1.record()
            torch.cuda.synchronize()
            t = torch.tensor([e0.elapsed_time(e1) / steps], device="cuda")
            if world > 1:
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return t.item()

        t_f = timed(lambda: sn.forward(x, gamma, out=y))
        t_b = timed(lambda: sn.backward(dy, x, gamma, reduce="none"))
        t_bg = timed(lambda: sn.backward(dy, x, gamma, reduce="ordered"))
        bf, bb = 4 * R * H + 4 * H, 6 * R * H + 8 * H
        out[f"h{H}"] = {"fwd_ms": t_f, "fwd_gbs": bf / t_f / 1e6, "bwd_local_dgamma_ms": t_b,
                        "bwd_local_dgamma_gbs": bb / t_b / 1e6, "bwd_global_dgamma_ms": t_bg,
                        "bwd_global_dgamma_gbs": bb / t_bg / 1e6,
                        "fwd_frac_of_measured_hbm_per_gpu": bf / t_f / 1e6 / world / peaks["hbm_gbs"],
                        "bwd_frac_of_measured_hbm_per_gpu": bb / t_b / 1e6 / world / peaks["hbm_gbs"]}
        del x, dy, y
    return out


def config5(args) -> None:
    """benchmark config 5: m = n = 32768, k = 16384 bf16, B column-sharded over the ranks (strong scaling),
    timed without a gather, with the all-gather (native shard-major result) and with the copy to row-major."""
    import torch
    import torch.distributed as dist

    from peakgemm_b200 import capi
    from peakgemm_b200.dist import ShardedGemm

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    m = n = 32768
    k = 16384
    sg = ShardedGemm(n)
    g = torch.Generator(device="cuda").manual_seed(4)
    a = (torch.rand(m, k, device="cuda", generator=g) * 2 - 1).to(torch.bfloat16)
    g.manual_seed(400 + rank)
    b = (torch.rand(sg.n_local, k, device="cuda", generator=g) * 2 - 1).to(torch.bfloat16)
    out = torch.empty(m, sg.n_local, dtype=torch.bfloat16, device="cuda")

    def timed(fn, steps):
        for _ in range(2):
            fn()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / steps], device="cuda")
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.item()

    res = {"n_gpus": world, "m": m, "n": n, "k": k, "flop": 2.0 * m * n * k}
    res["no_gather_ms"] = timed(lambda: sg.local(a, b, out=out), args.steps)
    if world > 1:
        for bands, max_sms in ((1, 0), (4, 0), (4, 140), (8, 132)):
            key = f"gather_shard_major_bands{bands}_sms{max_sms}_ms"
            res[key] = timed(lambda: sg.gathered(a, b, layout="shard_major", bands=bands, max_sms=max_sms),
                             max(2, args.steps // 2))
        res["gather_row_major_bands4_ms"] = timed(lambda: sg.gathered(a, b, layout="row_major", bands=4, max_sms=140),
                                                  max(2, args.steps // 2))
        from peakgemm_b200.dist import PeerMatrix

        pm = PeerMatrix(m, n, torch.bfloat16)
        res["gather_fused_row_major_ms"] = timed(lambda: sg.gathered_fused(pm, a, b), max(2, args.steps // 2))
    res["tflops_no_gather"] = res["flop"] / (res["no_gather_ms"] * 1e-3) / 1e12
    assert capi.device_status() == 0
    if rank == 0:
        print(json.dumps({"config5": res}))
    if world > 1:
        dist.destroy_process_group()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--variant", type=int, default=0, help="GEMM kernel variant (0 auto, 1 one-CTA, 2 CTA pair)")
    ap.add_argument("--block-n", type=int, default=0)
    ap.add_argument("--no-extras", action="store_true", help="skip comparators, RMSNorm, e2e and CPU legs")
    ap.add_argument("--size", type=int, default=8192,
                    help="m=n=k of the GEMM; anything but 8192 is a profiling case, not the headline workload")
    ap.add_argument("--shape", type=int, nargs=3, default=None, metavar=("M", "N", "K"),
                    help="profiling case: a non-square GEMM instead of the headline workload")
    ap.add_argument("--cublas", action="store_true",
                    help="with --no-extras: also run the cuBLAS comparator (torch.matmul) for the same steps after "
                         "the timed region, so that a profiler sees both kernels in one process")
    ap.add_argument("--config5", action="store_true",
                    help="benchmark config 5 (32768 x 32768 x 16384 sharded over the ranks, with and without the "
                         "all-gather); prints one JSON object and exits")
    ap.add_argument("--probe", action="store_true", help="run only the roofline probes; prints one JSON object and exits")
    ap.add_argument("--sweep", action="store_true",
                    help="benchmark configs 2 and 3 (every shape) against cuBLAS; prints one JSON object and exits")
    ap.add_argument("--chain", action="store_true",
                    help="RMSNorm -> projection chains (two operators, fused, fused + overlapped launch, torch); "
                         "prints one JSON object and exits")
    ap.add_argument("--only-rmsnorm", type=int, default=0, metavar="ROWS",
                    help="profiling case: run only the RMSNorm kernels on [ROWS, 4096] and [ROWS, 8192] and exit")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    global M, N, K, WORKLOAD
    if args.size != 8192:
        M = N = K = args.size
        WORKLOAD = f"PROFILING CASE bf16 GEMM m=n=k={args.size} TN (not the headline workload)"
    if args.shape:
        M, N, K = args.shape
        WORKLOAD = f"PROFILING CASE bf16 GEMM m={M} n={N} k={K} TN (not the headline workload)"

    if args.impl == "reference":
        run_reference_arm(args)
        return
    if args.config5:
        config5(args)
        return

    import torch
    import torch.distributed as dist

    import peakgemm_b200
    from peakgemm_b200 import capi

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    assert torch.cuda.is_available(), "bench.py needs a CUDA device: there is no CPU path"
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    peaks = measured_peaks()
    if args.probe:
        print(json.dumps({"probe": probes()}))
        return
    if args.sweep:
        print(json.dumps({"sweep": shape_sweep(peaks), "peaks": {k: v for k, v in peaks.items() if not isinstance(v, dict)}}))
        return
    if args.chain:
        print(json.dumps({"chain": chain_sweep()}))
        return
    if args.only_rmsnorm:
        print(json.dumps({"profiling_case": "rmsnorm", "rows": args.only_rmsnorm,
                          "rmsnorm": rmsnorm_numbers(peaks, args.steps, args.warmup, rows=args.only_rmsnorm)}))
        return

    # Inputs: generated on the device from seed 1 (the parity tests use CPU-generated copies of the
    # same distribution); rank r holds A and the r-th 8192-column block of B.
    g = torch.Generator(device="cuda").manual_seed(1)
    a = (torch.rand(M, K, device="cuda", generator=g) * 2 - 1).to(torch.bfloat16)
    g.manual_seed(1000 + rank)
    b = (torch.rand(N, K, device="cuda", generator=g) * 2 - 1).to(torch.bfloat16)
    c = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")

    def step():
        capi.hgemm(c, a, b, variant=args.variant, block_n=args.block_n)

    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local_rank) as clocks:
        e0.record()
        for _ in range(args.steps):
            step()
        e1.record()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        if args.steps * 1.0 < 400:          # keep the sampler alive long enough for a few samples
            t_end = time.time() + 0.5
            while time.time() < t_end:
                step()
            torch.cuda.synchronize()
    ms = torch.tensor([e0.elapsed_time(e1)], device="cuda")
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    total_ms = ms.item()
    ms_per_step = total_ms / args.steps
    flops_step = 2.0 * M * N * K
    value = world * flops_step / (ms_per_step * 1e-3) / 1e12
    assert capi.device_status() == 0, "a GEMM kernel abandoned a bounded wait"

    per_gpu = value / world
    peak_key = "bf16_tflops" if total_ms < 1000 else "bf16_tflops_sustained"
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": bench_config(world),
        "kernel": f"variant={args.variant} block_n={args.block_n} (0 = automatic)",
        "gpu_launches": args.steps,
        "roofline": {"bound": "tensor", "achieved": per_gpu, "peak": peaks[peak_key], "unit": "TFLOP/s",
                     "frac": per_gpu / peaks[peak_key],
                     "peak_source": f"{peaks['_source']} cuBLAS bf16 8192^3 ({peak_key})",
                     "frac_of_nominal_2250": per_gpu / 2250.0,
                     "traffic": ncu_traffic("hgemm_tcgen05_kernel_8192")},
    }

    if not args.no_extras:
        # ---- end to end through the torch operator with host buffers: every rank, max over ranks
        t_e2e, e2e_steps = e2e_ms(a, b, c, args.steps)
        t = torch.tensor([t_e2e], device="cuda")
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        t_e2e = t.item()
        line["e2e"] = {"value": world * flops_step / (t_e2e * 1e-3) / 1e12, "unit": UNIT, "ms_per_step": t_e2e,
                       "steps": e2e_steps, "h2d_bytes_per_step": world * 2 * (M * K + N * K),
                       "d2h_bytes_per_step": world * 2 * M * N,
                       "how": "PeakGemm.gemm_peak on pinned-host inputs: H2D of A and B, the operator, D2H of C every "
                              "step on every rank; 3 buffer sets on 3 streams so consecutive steps overlap on the "
                              "full-duplex link; max over ranks",
                       "pcie_in_gbs_per_gpu": 2 * (M * K + N * K) / (t_e2e * 1e-3) / 1e9}
    if rank == 0 and not args.no_extras and world == 1:
        # ---- the reference's own timing styles next to the steady-state figure
        line["reference_style_timing"] = reference_style_timing(a, b, c, flops_step)
        # ---- comparators on the same GPU and inputs (never on the product path)
        t_cublas = time_cuda(lambda: torch.matmul(a, b.t(), out=c), args.steps, args.warmup)
        line["cublas"] = {"tflops": flops_step / (t_cublas * 1e-3) / 1e12, "ms": t_cublas}
        ref_path = os.path.join(REPO, "oracle", "_ref", "libref_peakgemm.so")
        if os.path.exists(ref_path):
            ref = ctypes.CDLL(ref_path)
            ref.ref_hgemm_peak.argtypes = [ctypes.c_void_p] * 3 + [ctypes.c_uint] * 3 + [ctypes.c_int, ctypes.c_void_p]
            s = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
            t_ref = time_cuda(lambda: ref.ref_hgemm_peak(c.data_ptr(), a.data_ptr(), b.data_ptr(), M, N, K, 1, s),
                              min(args.steps, 10), 3)
            line["reference_kernel_on_this_gpu"] = {"tflops": flops_step / (t_ref * 1e-3) / 1e12, "ms": t_ref,
                                                    "what": "reference mma.sync hgemm_peak compiled for sm_100a"}
        line["rmsnorm"] = rmsnorm_numbers(peaks, args.steps, args.warmup)
        line["cpu_baseline"] = cpu_gemm_baseline()
    if args.no_extras and args.cublas and world == 1:
        t_cublas = time_cuda(lambda: torch.matmul(a, b.t(), out=c), args.steps, args.warmup)
        line["cublas"] = {"tflops": flops_step / (t_cublas * 1e-3) / 1e12, "ms": t_cublas}
    if not args.no_extras and args.size == 8192 and not args.shape:
        # ---- the multi-GPU split of the sharded benchmark shape on the same ranks (N = 1: its denominator)
        del a, b, c
        torch.cuda.empty_cache()
        line["config5"] = config5_block(world, rank)
        line["rmsnorm_sharded"] = rmsnorm_sharded_block(world, rank, peaks)
    line["clocks"] = clocks.summary()

    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
