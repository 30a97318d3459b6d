#!/usr/bin/env python
"""Benchmark of the TCEC SGEMM hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--size S] [--only kernel]

N = 1.  One step = one error-corrected SGEMM, C = A * B, M = N = K = S (default 16384, the
size the throughput target is stated at), FP32 row-major operands, through the public call
(split of both operands + three-product tcgen05 GEMM), fp16 hi/lo policy on U[-1,1) values.
Beside the headline the line carries: the same shape with the wide-exponent values
sign * U[1,2) * 2^U{-15..15} (tf32 policy accurate, fp16 heads overflow), the 4096^3 configuration
with its full-matrix error, the 65536 x 65536 x 8192 configuration on one GPU (the anchor of the
multi-GPU runs), the batched configuration, the reference's own GPU kernel on the same box, and
the end-to-end figure from pinned host memory through tcec_sgemm_host.

N > 1 (launched by torchrun, one rank per GPU).  One step = the large configuration
M = N = 65536, K = 8192, N(0,1) values, strong-scaled: B and C are divided into column blocks of
whole output tiles, A (2 GiB, on rank 0) is broadcast by NCCL inside the timed region
(tcec_sgemm_column_shard).  Every rank checks sampled rows of its block against the FP64 host loop.

Throughput is FP32-equivalent: 2*M*N*K flop per GEMM.

--impl reference times the reference's CPU path, its FP64 host check loop
(test/tcec/batch_gemm.cu:561-575), ported in oracle/tcec_oracle.c, on a bounded row sample of the
same workload with all host cores.  --only kernel runs nothing but the headline GEMM of N = 1,
--only batched nothing but the batched configuration (the commands the profiler captures are made with).
"""
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

METRIC = "tcec_sgemm_fp32_equiv_tflops"
UNIT = "TFLOP/s"


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"bf16_burst": d["bf16_tflops"], "bf16_sustained": d.get("bf16_tflops_sustained", d["bf16_tflops"]),
                "hbm_gbs": d["hbm_gbs"], "source": "measured (MEASURED_PEAKS.json)"}
    return {"bf16_burst": 1590.0, "bf16_sustained": 1400.0, "hbm_gbs": 6650.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clock, power and throttle reasons while the timed region runs: NVML from a
    thread every 10 ms (read-only queries), or nvidia-smi every 100 ms where NVML is missing."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")
    NAMES = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.nvml = None
        self.samples = []  # (sm_mhz, sm_max_mhz, power_w, set(reasons))
        self.first = 0
        self.last = None
        self._stop = False

    def start(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(self.index)
            self.smax = pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM)
            self.nvml = pynvml
            self.thread = threading.Thread(target=self._poll_nvml, daemon=True)
            self.thread.start()
        except Exception:
            self.nvml = None
            try:
                self.proc = subprocess.Popen(
                    ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                     "--format=csv,noheader,nounits", "-lms", "100"],
                    stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
                self.thread = threading.Thread(target=self._read_smi, daemon=True)
                self.thread.start()
            except OSError:
                self.proc = None
        t0 = time.time()
        while not self.samples and time.time() - t0 < 5.0:
            time.sleep(0.02)

    def _poll_nvml(self):
        n = self.nvml
        masks = {"hw_slowdown": 0x8, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20, "sw_power_cap": 0x4}
        while not self._stop:
            try:
                clk = n.nvmlDeviceGetClockInfo(self.handle, n.NVML_CLOCK_SM)
                pw = n.nvmlDeviceGetPowerUsage(self.handle) / 1000.0
                try:
                    bits = n.nvmlDeviceGetCurrentClocksEventReasons(self.handle)
                except Exception:
                    bits = n.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle)
                self.samples.append((float(clk), float(self.smax), pw, {k for k, m in masks.items() if bits & m}))
            except Exception:
                pass
            time.sleep(0.01)

    def _read_smi(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                rec = (float(parts[0]), float(parts[1]), float(parts[2]),
                       {nm for nm, val in zip(self.NAMES, parts[3:7]) if val.lower().startswith("active")})
            except ValueError:
                continue
            self.samples.append(rec)

    def mark_begin(self):
        self.first = len(self.samples)

    def mark_end(self):
        self.last = len(self.samples)

    def stop(self):
        self._stop = True
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        if self.nvml is None and self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        window = self.samples[self.first:self.last] if self.last and self.last > self.first else self.samples
        sm = [w[0] for w in window]
        reasons = set()
        for w in window:
            reasons |= w[3]
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(w[1] for w in window) if window else None,
                "power_w_max": max(w[2] for w in window) if window else None,
                "reasons": sorted(reasons), "samples": len(sm),
                "source": "nvml 10 ms" if self.nvml is not None else "nvidia-smi 100 ms"}


def make_uniform(torch, device, rows, cols, seed):
    """U[-1, 1) values."""
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    return torch.rand((rows, cols), generator=g, device=device) * 2.0 - 1.0


def make_normal(torch, device, rows, cols, seed):
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    return torch.randn((rows, cols), generator=g, device=device)


def make_wide(torch, device, rows, cols, seed):
    """sign * U[1,2) * 2^e, e uniform integer in -15..15."""
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    mant = 1.0 + torch.rand((rows, cols), generator=g, device=device)
    expo = torch.randint(-15, 16, (rows, cols), generator=g, device=device).to(torch.float32)
    sign = torch.where(torch.rand((rows, cols), generator=g, device=device) < 0.5, -1.0, 1.0)
    return sign * mant * torch.exp2(expo)


LARGE = (65536, 65536, 8192)  # M, N, K of the column-sharded configuration


def bench_config(world, size, large, panel_rows):
    """The `config` object of the JSON line: the same for both arms of a run."""
    if world == 1:
        return {"workload": f"sgemm M=N=K={size}, FP32 row-major A,B, U[-1,1), alpha=1 beta=0, one GPU",
                "policy": "fp16_ec", "parallelism": "single GPU",
                "l2": "operands (1 GiB each at 16384) exceed the 126 MB L2; no flush needed"}
    m, n, k = large
    return {"workload": f"sgemm M={m} N={n} K={k}, FP32 row-major A,B, N(0,1), alpha=1 beta=0, strong-scaled over "
                        f"{world} GPUs",
            "policy": "fp16_ec",
            "parallelism": f"B and C in column blocks of whole 256-column tiles over {world} GPUs; A ({m * k * 4 >> 20} MiB, on "
                           f"rank 0) split once and broadcast by NCCL in {panel_rows}-row panels inside the timed region",
            "l2": "every operand exceeds the 126 MB L2; no flush needed"}


def cpu_baseline_sample(k, n, what, seconds=12.0, seed=3, normal=False):
    """Times the FP64 host loop on rows of A against the full k x n B; returns (dict, rows, seconds)."""
    import numpy as np

    from oracle import cpu

    cores = cpu.use_all_cores()
    rng = np.random.default_rng(seed)

    def gen(shape):
        if normal:
            return rng.standard_normal(shape, dtype=np.float32)
        return (rng.random(shape, dtype=np.float32) * 2 - 1).astype(np.float32)

    b = gen((k, n))
    probe_rows = max(cores, 8)
    a = gen((probe_rows, k))
    t0 = time.perf_counter()
    cpu.gemm_f64(a, b)
    dt = time.perf_counter() - t0
    rows = int(max(probe_rows, probe_rows * seconds / max(dt, 1e-3)))
    rows = (rows // cores) * cores or probe_rows
    a = gen((rows, k))
    t0 = time.perf_counter()
    cpu.gemm_f64(a, b)
    dt = time.perf_counter() - t0
    tf = 2.0 * rows * k * n / dt * 1e-12
    return {"value": tf, "unit": UNIT, "cores": cores, "kind": "port",
            "sample": f"{rows} rows of A against the full {k}x{n} B of {what}, FP64 host loop with OpenMP on {cores} "
                      f"threads ({dt:.1f} s)"}, rows, dt


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    world = args.gpus
    large = tuple(args.large)
    if world == 1:
        k, n, what, normal = args.size, args.size, f"M=N=K={args.size}", False
    else:
        k, n, what, normal = large[2], large[1], f"M={large[0]} N={large[1]} K={large[2]}", True
    times = []
    base = None
    for i in range(args.warmup + args.steps):
        base, rows, dt = cpu_baseline_sample(k, n, what, seconds=max(2.0, 20.0 / max(1, args.steps + args.warmup)),
                                            normal=normal)
        if i >= args.warmup:
            times.append((rows, dt))
    flop = sum(2.0 * r * k * n for r, _ in times)
    secs = sum(dt for _, dt in times)
    value = flop / secs * 1e-12
    base["value"] = value
    line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": secs / max(1, len(times)) * 1e3, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f64", "data": "synthetic", "impl": "reference",
            "config": bench_config(world, args.size, large, args.panel_rows),
            "reference_arm_is": "the reference's CPU path: its FP64 host check loop (test/tcec/batch_gemm.cu:561-575)",
            "cpu_baseline": base,
            "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def time_loop(torch, fn, steps, dist_on):
    """K calls between two events on the current stream; barrier + sync on both sides."""
    if dist_on:
        import torch.distributed as dist
        dist.barrier()
    torch.cuda.synchronize()
    e0 = torch.cuda.Event(enable_timing=True)
    e1 = torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    if dist_on:
        import torch.distributed as dist
        dist.barrier()
    return e0.elapsed_time(e1)


def per_step_times(torch, fn, steps):
    """Device time of each of `steps` calls (an event pair per call); for best / median beside the loop's mean."""
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    torch.cuda.synchronize()
    for e0, e1 in ev:
        e0.record()
        fn()
        e1.record()
    torch.cuda.synchronize()
    return sorted(e0.elapsed_time(e1) for e0, e1 in ev)


def error_metrics(torch, c, exact):
    """The three error forms of the reference's tests against an FP64 product of the whole matrix: max |d| / max |ref|
    (test/primitive/common.hpp:100-102), relative Frobenius residual (test/tcec/batch_gemm.cu:605), max |d|
    (test/tcec/mma.cu:152).  Non-finite elements of c (fp16 heads that overflowed) are left out and counted."""
    finite = torch.isfinite(c)
    d = torch.where(finite, c.double() - exact, torch.zeros_like(exact))
    out = {"max_rel": (d.abs().max() / exact.abs().max()).item(),
           "fro_rel": (torch.linalg.norm(d) / torch.linalg.norm(exact)).item(), "max_abs": d.abs().max().item()}
    nf = 1.0 - finite.double().mean().item()
    if nf:
        out["nonfinite_fraction"] = nf
    return out


def max_over_ranks(torch, value, device, dist_on):
    if not dist_on:
        return value
    import torch.distributed as dist
    t = torch.tensor([value], device=device, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.item()


def bind_to_gpu_numa_node(index):
    """Runs this process on the CPUs next to its GPU, so that the pinned buffers it allocates
    afterwards are placed on that NUMA node (host-side scheduling only; no GPU setting changes)."""
    try:
        import pynvml
        pynvml.nvmlInit()
        h = pynvml.nvmlDeviceGetHandleByIndex(index)
        words = (os.cpu_count() + 63) // 64
        mask = pynvml.nvmlDeviceGetCpuAffinity(h, words)
        cpus = [64 * w + b for w, bits in enumerate(mask) for b in range(64) if (bits >> b) & 1]
        if cpus:
            os.sched_setaffinity(0, cpus)
            return len(cpus)
    except Exception:
        pass
    return 0


def sampled_accuracy(torch, np, cpu, a_rows, b_dev, c_rows):
    """max|d|, max|ref| and the FP32-FMA loop's max|d| of sampled rows against the FP64 host loop."""
    b_host = b_dev.cpu().numpy()
    exact = cpu.gemm_f64(a_rows, b_host)
    got = c_rows.cpu().numpy()
    finite = np.isfinite(got)
    d = np.abs(np.where(finite, got, 0).astype(np.float64) - np.where(finite, exact, 0))
    d32 = np.abs(cpu.gemm_f32(a_rows, b_host).astype(np.float64) - exact)
    return float(d.max()), float(np.abs(exact).max()), float(d32.max()), float(1.0 - finite.mean())


def np_sample(count, how_many, seed):
    import numpy as np

    if count <= how_many:
        return list(range(count))
    return [int(i) for i in np.random.default_rng(seed).choice(count, size=how_many, replace=False)]


def batched_extra(torch, tcec, sharded, peaks, args, rank, world, device, dist_on):
    """8192 independent 256^3 products, N(0,1), batch-sharded (no collective); strong scaling."""
    nb, bs = args.batched, 256
    first, count = sharded.batch_shard(nb, rank, world)
    g = torch.Generator(device=device)
    g.manual_seed(4000 + rank)
    ab = torch.randn((count, bs, bs), generator=g, device=device)
    bb = torch.randn((count, bs, bs), generator=g, device=device)
    cb = torch.empty((count, bs, bs), dtype=torch.float32, device=device)
    for _ in range(3):
        sharded.sgemm_batch_sharded(ab, bb, cb, policy="fp16_ec")
    ms_b = time_loop(torch, lambda: sharded.sgemm_batch_sharded(ab, bb, cb, policy="fp16_ec"), args.steps, dist_on)
    ms_b = max_over_ranks(torch, ms_b, device, dist_on) / args.steps
    # 64 whole matrices of this rank's shard (first, last and a seeded sample) against FP64 products
    pick = sorted({0, count - 1, *np_sample(count, 62, 4100 + rank)}) if count > 0 else []
    idx = torch.tensor(pick, device=device, dtype=torch.long)
    ref_b = torch.matmul(ab[idx].double(), bb[idx].double())
    d_b = (cb[idx].double() - ref_b).abs()
    scale_b = ref_b.abs().amax(dim=(1, 2))
    err_b = (d_b.amax(dim=(1, 2)) / scale_b).max().item()
    fro_b = (torch.linalg.norm(d_b.flatten(1), dim=1) / torch.linalg.norm(ref_b.flatten(1), dim=1)).max().item()
    abs_b = d_b.max().item()
    t = torch.tensor([err_b, fro_b, abs_b], device=device, dtype=torch.float64)
    if dist_on:
        import torch.distributed as dist
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    err_b, fro_b, abs_b = t.tolist()
    tcec.device_status()
    flop_b = 2.0 * bs ** 3 * nb
    hbm_cap = (2.0 * bs ** 3) / (3 * bs * bs * 4) * peaks["hbm_gbs"] * 1e-3 * world  # flop/B x GB/s, all ranks
    return {"workload": f"{nb} x ({bs}x{bs}x{bs}), N(0,1), fp16_ec, batch-sharded over {world} GPU(s) (strong scaling, no "
                        "collective)",
            "tflops": flop_b / (ms_b * 1e-3) * 1e-12, "ms_per_call": ms_b, "hbm_roofline_tflops": hbm_cap,
            "frac_of_hbm_roofline": flop_b / (ms_b * 1e-3) * 1e-12 / hbm_cap, "max_rel_err_sampled": err_b,
            "errors_sampled_matrices": {"matrices_per_rank": 64, "max_rel": err_b, "fro_rel": fro_b, "max_abs": abs_b,
                                        "how": "first, last and 62 seeded matrices of every rank's shard against GPU FP64 "
                                               "products; maxima over matrices and ranks"},
            "kernel": "tcec_gemm_fused_kernel<ec> (CTA pairs)"}


# DRAM traffic of one launch of tcec_gemm_panels_kernel<256,fp16,ec> on M = N = K = size, from ncu captures
# (dram__bytes_read.sum + dram__bytes_write.sum; profiles/): C is written once, A's panels are read about
# once per pass, and B's panels once per group of 2048 rows of A, because neither operand fits the L2.
TRAFFIC_POINTS = {6144: 1.130e9, 8192: 2.535e9, 16384: 37.2e9}


def panel_gemm_traffic(size):
    if size in TRAFFIC_POINTS:
        return TRAFFIC_POINTS[size], "measured"
    s0 = max(TRAFFIC_POINTS)
    # bytes = 4 s^2 (c0 + c1 s / 2048): fitted through the captured points (one point: c0 = 2, the A and C terms)
    if len(TRAFFIC_POINTS) >= 2:
        (sa, ta), (sb, tb) = sorted(TRAFFIC_POINTS.items())[-2:]
        ya, yb = ta / (4.0 * sa * sa), tb / (4.0 * sb * sb)
        c1 = (yb - ya) / ((sb - sa) / 2048.0)
        c0 = ya - c1 * sa / 2048.0
    else:
        c0 = 2.0
        c1 = (TRAFFIC_POINTS[s0] / (4.0 * s0 * s0) - c0) / (s0 / 2048.0)
    return 4.0 * size * size * (c0 + c1 * size / 2048.0), "fitted"


def run_single(args, torch, np, tcec, sharded, peaks, device):
    from oracle import cpu, ref

    rank, world, dist_on = 0, 1, False
    if args.only == "batched":
        print(json.dumps({"metric": METRIC, "n_gpus": 1, "steps": args.steps,
                          "batched_256": batched_extra(torch, tcec, sharded, peaks, args, 0, 1, device, False)}), flush=True)
        return
    size = args.size
    m = n = k = size
    policy = args.policy if args.only == "kernel" else "fp16_ec"
    tf32_peak = None
    if args.only != "kernel":
        # ---- measured dense tf32 throughput of the box (cuBLAS through torch), for the tf32 policy's roofline: a burst
        #      figure like the 16-bit one of MEASURED_PEAKS.json, so it is taken first, before the long loops heat the GPU
        x = torch.randn((8192, 8192), device=device)
        y = torch.randn((8192, 8192), device=device)
        prev = torch.backends.cuda.matmul.allow_tf32
        torch.backends.cuda.matmul.allow_tf32 = True
        for _ in range(3):
            torch.matmul(x, y)
        best = min(time_loop(torch, lambda: torch.matmul(x, y), 1, False) for _ in range(10))
        torch.backends.cuda.matmul.allow_tf32 = prev
        tf32_peak = 2.0 * 8192 ** 3 / (best * 1e-3) * 1e-12
        del x, y
        # ---- 4096^3, U[-1,1): the small square configuration is a 0.36 ms call, timed here, before the long loops
        #      (its errors are taken further down, with the other comparators)
        s2 = 4096
        a2, b2 = make_uniform(torch, device, s2, s2, seed=2), make_uniform(torch, device, s2, s2, seed=1002)
        c2 = torch.empty((s2, s2), device=device)
        for _ in range(5):
            tcec.sgemm(a2, b2, c2, policy=policy)
        reps2 = max(10, args.steps)
        ms2 = time_loop(torch, lambda: tcec.sgemm(a2, b2, c2, policy=policy), reps2, False) / reps2
        t2 = per_step_times(torch, lambda: tcec.sgemm(a2, b2, c2, policy=policy), reps2)
        del a2, b2, c2
    a = make_uniform(torch, device, m, k, seed=3)
    b = make_uniform(torch, device, k, n, seed=1003)
    c = torch.empty((m, n), dtype=torch.float32, device=device)
    flop = 2.0 * m * n * k

    def step():
        tcec.sgemm(a, b, c, policy=policy)

    for _ in range(max(args.warmup, 3)):
        step()
    tcec.device_status()

    # The dominant kernel's duration, for the roofline: the step's own work (split of A, split of B, GEMM:
    # tcec_pack_a / tcec_pack_b / tcec_sgemm_packed run what tcec_sgemm runs, the two splits as two launches
    # instead of one), back to back, with an event pair around each GEMM launch.  The GPU keeps heating through
    # the run (later loops come out a few percent slower), so this loop runs directly before and directly after
    # the timed region and the two means are averaged.
    ap = bp = None

    def gemm_launch_ms(nsteps):
        ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(nsteps)]
        torch.cuda.synchronize()
        for e0, e1 in ev:
            tcec.pack_a(a, policy, out=ap)
            tcec.pack_b(b, policy, out=bp)
            e0.record()
            tcec.sgemm_packed(ap, bp, m, n, k, c, policy=policy)
            e1.record()
        torch.cuda.synchronize()
        return sum(e0.elapsed_time(e1) for e0, e1 in ev) / nsteps

    ms_k_before = None
    if args.only != "kernel":
        ap, bp = tcec.pack_a(a, policy), tcec.pack_b(b, policy)
        tcec.sgemm_packed(ap, bp, m, n, k, c, policy=policy)
        ms_k_before = gemm_launch_ms(min(args.steps, 2))  # short: it must not heat the GPU for the timed region
    sampler = ClockSampler(device.index)
    sampler.start()
    for _ in range(2):
        step()
    torch.cuda.synchronize()
    sampler.mark_begin()
    ms = time_loop(torch, step, args.steps, False)
    sampler.mark_end()
    clocks = sampler.stop()
    tcec.device_status()
    ms_per_step = ms / args.steps
    value = flop / (ms_per_step * 1e-3) * 1e-12
    line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": 1, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f16 hi/lo products, f32 accumulate",
            "data": "synthetic", "config": bench_config(1, size, tuple(args.large), args.panel_rows),
            "clocks": clocks, "gpu_launches": 2 * args.steps}  # the split of A and B (one launch), the GEMM
    line["config"]["promote_k"] = tcec.get_option("promote_k")
    line["config"]["policy"] = policy
    if args.only == "kernel":
        print(json.dumps(line), flush=True)
        return

    ms_k_after = gemm_launch_ms(args.steps)
    ms_k = 0.5 * (ms_k_before + ms_k_after) * args.steps
    achieved = flop / (ms_k / args.steps * 1e-3) * 1e-12
    del ap, bp
    peak = peaks["bf16_burst"] / 3.0
    traffic, how = panel_gemm_traffic(size)
    line["roofline"] = {
        "bound": "tensor", "achieved": achieved, "peak": peak, "unit": UNIT, "frac": achieved / peak,
        "traffic": traffic,
        "traffic_is": f"dram__bytes_read+write of one launch of this kernel, {how} from the ncu captures in profiles/",
        "peak_is": f"dense 16-bit tensor peak (burst) / 3 products, {peaks['source']}",
        "frac_of_sustained_peak": achieved / (peaks["bf16_sustained"] / 3.0),
        "sustained_is": "the same with the sustained dense figure: this kernel runs ~20 ms per launch, back to back, at "
                        "the board's power cap",
        "kernel": "tcec_gemm_panels_kernel<256,fp16,ec>", "kernel_ms": ms_k / args.steps,
        "kernel_timed": "an event pair around each GEMM launch of full steps (split A, split B, GEMM) run back to back, "
                        "in a short loop (two steps) directly before and a loop directly after the timed region; the mean of the two",
        "kernel_ms_before": ms_k_before, "kernel_ms_after": ms_k_after}

    # ---- accuracy of the headline on sampled rows (outside any timed region)
    rows = [0, 1, m // 2 - 1, m // 2, m - 1]

    def errors_of(aa, bb, pol):
        tcec.sgemm(aa, bb, c, policy=pol)
        dmax, rmax, d32, nonfinite = sampled_accuracy(torch, np, cpu, aa[rows].cpu().numpy(), bb, c[rows])
        return dmax / rmax, nonfinite, d32 / rmax

    e_h, nf_h, e_f = errors_of(a, b, policy)
    line["accuracy"] = {"rows_checked": len(rows), "max_rel": e_h, "fp16_ec_max_rel": e_h, "fp32_fma_max_rel": e_f,
                        "nonfinite_fraction": nf_h}
    # the whole matrix against a GPU FP64 product, for this library and for cuBLAS FP32 on the same inputs
    exact = a.double() @ b.double()
    line["accuracy"]["full_matrix_vs_gpu_fp64"] = {policy: error_metrics(torch, c, exact)}
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.matmul(a, b, out=c)
    torch.backends.cuda.matmul.allow_tf32 = prev
    line["accuracy"]["full_matrix_vs_gpu_fp64"]["cublas_fp32"] = error_metrics(torch, c, exact)
    del exact
    # best and median of single calls, beside the mean of the timed loop
    t = per_step_times(torch, step, max(10, args.steps))
    line["ms_per_step_best"], line["ms_per_step_median"] = t[0], t[len(t) // 2]

    # ---- same shape, wide-exponent values: tf32 policy (accurate) vs fp16 policy (heads overflow)
    aw, bw = make_wide(torch, device, m, k, seed=3), make_wide(torch, device, k, n, seed=1003)
    wide = {"values": "sign*U[1,2)*2^U{-15..15}"}
    for pol in ("tf32_ec", "fp16_ec"):
        for _ in range(2):
            tcec.sgemm(aw, bw, c, policy=pol)
        st = max(2, args.steps // 2)
        ms_t = time_loop(torch, lambda: tcec.sgemm(aw, bw, c, policy=pol), st, False)
        e, nf, e32 = errors_of(aw, bw, pol)
        wide[pol] = {"tflops": flop / (ms_t / st * 1e-3) * 1e-12, "max_rel_err_finite": e, "nonfinite_fraction": nf}
        wide["fp32_fma_max_rel"] = e32
        exact = aw.double() @ bw.double()
        wide[pol]["full_matrix_vs_gpu_fp64"] = error_metrics(torch, c, exact)  # c still holds errors_of's product
        del exact
    wide["tf32_dense_peak_measured"] = tf32_peak
    wide["tf32_ec"]["frac_of_tf32_roofline"] = wide["tf32_ec"]["tflops"] / (tf32_peak / 3.0)
    wide["tf32_roofline_is"] = "dense tf32 throughput measured in this run (torch.matmul with TF32 allowed, 8192^3, best " \
                               "of 10) / 3 products"
    line["wide_exponent"] = wide
    del aw, bw

    # ---- end to end from pinned host buffers through the C entry for host operands
    bind_to_gpu_numa_node(device.index)
    ah = torch.empty((m, k), dtype=torch.float32, pin_memory=True)
    bh = torch.empty((k, n), dtype=torch.float32, pin_memory=True)
    ch = torch.empty((m, n), dtype=torch.float32, pin_memory=True)
    ah.copy_(a)
    bh.copy_(b)
    torch.cuda.synchronize()

    def e2e_step():
        tcec.sgemm_host(ah, bh, ch, policy=policy)  # automatic panel height

    e2e_step()
    tcec.sgemm(a, b, c, policy=policy)
    torch.cuda.synchronize()
    e2e_ok = bool(torch.equal(ch[-256:], c[-256:].cpu()))
    e2e_steps = max(2, min(args.steps, 4))
    ms_e = time_loop(torch, e2e_step, e2e_steps, False)
    line["e2e"] = {"value": flop / (ms_e / e2e_steps * 1e-3) * 1e-12, "unit": UNIT,
                   "h2d_bytes_per_step": 4 * (m * k + k * n), "d2h_bytes_per_step": 4 * m * n,
                   "ms_per_step": ms_e / e2e_steps, "matches_device_resident_result": e2e_ok,
                   "how": "tcec_sgemm_host: pinned host A, B, C; B copied and split once, A in row panels; copy-in, GEMM "
                          "and copy-out overlapped on three streams"}
    del ah, bh, ch, a, b, c
    tcec.device_status()

    # ---- 4096^3, U[-1,1): the small square configuration, with the error of the whole matrix
    s2 = 4096
    a2, b2 = make_uniform(torch, device, s2, s2, seed=2), make_uniform(torch, device, s2, s2, seed=1002)
    c2 = torch.empty((s2, s2), device=device)
    tcec.sgemm(a2, b2, c2, policy=policy)
    exact = a2.double() @ b2.double()
    scale = exact.abs().max()
    m_ours = error_metrics(torch, c2, exact)
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    m_f32 = error_metrics(torch, a2 @ b2, exact)
    torch.backends.cuda.matmul.allow_tf32 = prev
    line["square_4096"] = {"workload": "sgemm M=N=K=4096, FP32 row-major, U[-1,1), fp16_ec (both splits + GEMM per call; timed "
                                       "first in the run, ten calls back to back after five warm-up calls)",
                           "tflops": 2.0 * s2 ** 3 / (ms2 * 1e-3) * 1e-12, "ms_per_call": ms2,
                           "ms_best": t2[0], "ms_median": t2[len(t2) // 2],
                           "frac_of_roofline": 2.0 * s2 ** 3 / (ms2 * 1e-3) * 1e-12 / peak,
                           "max_rel_err_full_matrix": m_ours["max_rel"], "cublas_fp32_max_rel_err": m_f32["max_rel"],
                           "errors_full_matrix": {"fp16_ec": m_ours, "cublas_fp32": m_f32}}
    tcec.sgemm(a2, b2, c2, policy="tf32_ec")
    line["square_4096"]["errors_full_matrix"]["tf32_ec"] = error_metrics(torch, c2, exact)
    # ---- the reference's own kernel (test/tcec/batch_gemm.cu:261-386 built for sm_100a) on the same box and
    #      inputs: the checker's library, run here only as a comparator, outside every timed region of this library
    if ref.available():
        refgpu = {"what": "the reference's bgemm_kernel (1024 CTAs), same 4096^3 inputs, device-timed"}
        for name, tf32 in (("fp16_ec", False), ("tf32_ec", True)):
            ref.bgemm(a2[None], b2[None], tf32=tf32, per=32)
            t0 = torch.cuda.Event(enable_timing=True)
            t1 = torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            t0.record()
            cr = ref.bgemm(a2[None], b2[None], tf32=tf32, per=32)[0]
            t1.record()
            torch.cuda.synchronize()
            msr = t0.elapsed_time(t1)  # includes the harness's transposed copy of B (a few percent)
            refgpu[name] = {"tflops": 2.0 * s2 ** 3 / (msr * 1e-3) * 1e-12, "ms": msr,
                            "max_rel_err_full_matrix": ((cr.double() - exact).abs().max() / scale).item(),
                            "errors_full_matrix": error_metrics(torch, cr, exact)}
        line["reference_gpu"] = refgpu
        # ... and at the headline size (16384 = 128 CTA tiles of 128 each way), fp16 policy, timed once after one warm-up
        try:
            ah16 = make_uniform(torch, device, size, size, seed=3)
            bh16 = make_uniform(torch, device, size, size, seed=1003)
            ref.bgemm(ah16[None], bh16[None], tf32=False, per=size // 128)
            t0 = torch.cuda.Event(enable_timing=True)
            t1 = torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            t0.record()
            cr = ref.bgemm(ah16[None], bh16[None], tf32=False, per=size // 128)[0]
            t1.record()
            torch.cuda.synchronize()
            msr = t0.elapsed_time(t1)
            refgpu["headline_size_fp16_ec"] = {"workload": f"M=N=K={size}, the headline's inputs", "ms": msr,
                                               "tflops": 2.0 * size ** 3 / (msr * 1e-3) * 1e-12}
            del ah16, bh16, cr
        except Exception as e:  # the harness has no instantiation for this size
            refgpu["headline_size_fp16_ec"] = {"unavailable": str(e)[:200]}
    del a2, b2, c2, exact
    tcec.device_status()

    # ---- the large configuration on one GPU: the anchor of the multi-GPU runs
    lm, ln_, lk = args.large
    free, _ = torch.cuda.mem_get_info()
    need = 4 * (lm * lk + lk * ln_ + lm * ln_) + 8 * (lm * lk + lk * ln_) + (2 << 30)
    if free > need:
        al = make_normal(torch, device, lm, lk, seed=5)
        bl = make_normal(torch, device, lk, ln_, seed=1005)
        cl = torch.empty((lm, ln_), device=device)
        for _ in range(2):
            tcec.sgemm(al, bl, cl, policy=policy)
        reps = 3
        msl = time_loop(torch, lambda: tcec.sgemm(al, bl, cl, policy=policy), reps, False) / reps
        rows = [0, 1, lm // 2 - 1, lm // 2, lm - 1]
        dmax, rmax, d32, _ = sampled_accuracy(torch, np, cpu, al[rows].cpu().numpy(), bl, cl[rows])
        line["large_single_gpu"] = {"workload": f"sgemm M={lm} N={ln_} K={lk}, N(0,1), fp16_ec, one GPU (both splits + GEMM per "
                                                "call)",
                                    "tflops": 2.0 * lm * ln_ * lk / (msl * 1e-3) * 1e-12, "ms_per_call": msl,
                                    "frac_of_roofline": 2.0 * lm * ln_ * lk / (msl * 1e-3) * 1e-12 / peak,
                                    "max_rel": dmax / rmax, "fp32_fma_max_rel": d32 / rmax, "rows_checked": len(rows)}
        del al, bl, cl
        tcec.device_status()

    line["batched_256"] = batched_extra(torch, tcec, sharded, peaks, args, rank, world, device, dist_on)
    line["cpu_baseline"], _, _ = cpu_baseline_sample(size, size, f"M=N=K={size}", seconds=12.0)
    print(json.dumps(line), flush=True)


def run_sharded(args, torch, np, tcec, sharded, peaks, device, rank, world):
    import torch.distributed as dist

    from oracle import cpu

    m, n, k = args.large
    policy = "fp16_ec"
    c0, cn = sharded.column_shard(n, rank, world)
    a = make_normal(torch, device, m, k, seed=5) if rank == 0 else None
    b = make_normal(torch, device, k, cn, seed=1005 + rank)
    c = torch.empty((m, cn), dtype=torch.float32, device=device)
    sharded.init_library_comm()
    flop = 2.0 * m * n * k
    panels = (m + args.panel_rows - 1) // args.panel_rows
    tcec.set_option("comm_panel_rows", args.panel_rows)

    def step():
        sharded.sgemm_column_sharded(a, b, c, m, k, root=0, policy=policy)

    for _ in range(max(args.warmup, 3)):
        step()
    tcec.device_status()
    sampler = ClockSampler(device.index)
    if rank == 0:
        sampler.start()
    for _ in range(2):  # every rank: the steps contain collectives
        step()
    torch.cuda.synchronize()
    if rank == 0:
        sampler.mark_begin()
    ms = time_loop(torch, step, args.steps, True)
    if rank == 0:
        sampler.mark_end()
    clocks = sampler.stop() if rank == 0 else None
    tcec.device_status()
    ms_per_step = max_over_ranks(torch, ms, device, True) / args.steps
    value = flop / (ms_per_step * 1e-3) * 1e-12

    # ---- the same per-rank product with A already on every GPU and nothing communicated: what the step
    #      would take if the broadcast and the root's split of A cost nothing (same clocks, same process)
    a_all = a if rank == 0 else torch.empty((m, k), dtype=torch.float32, device=device)
    dist.broadcast(a_all, src=0)
    c_chk = torch.empty_like(c)
    for _ in range(2):
        tcec.sgemm(a_all, b, c_chk, policy=policy)
    ms_local = max_over_ranks(torch, time_loop(torch, lambda: tcec.sgemm(a_all, b, c_chk, policy=policy), args.steps,
                                               True), device, True) / args.steps
    step()
    torch.cuda.synchronize()
    same_bits = torch.tensor([1.0 if torch.equal(c, c_chk) else 0.0], device=device, dtype=torch.float64)
    dist.all_reduce(same_bits, op=dist.ReduceOp.MIN)
    ms_again = max_over_ranks(torch, time_loop(torch, step, args.steps, True), device, True) / args.steps
    comm = {"sharded_step_ms": ms_again, "local_product_ms": ms_local, "ratio": ms_local / ms_again,
            "bit_identical_to_local_product": bool(same_bits.item() == 1.0),
            "what": "per rank, A already resident and nothing communicated (tcec_sgemm on the rank's block) against the "
                    "sharded step, both timed again back to back in this process: the cost of the split of A on the root, "
                    "the broadcast and the SMs left to it"}
    # ---- 64 seeded rows and 64 seeded columns of every rank's C block against GPU FP64 products (A is on every
    #      rank here), in the three error forms; c holds the sharded step's result
    ri = torch.tensor(sorted({0, m - 1, *np_sample(m, 62, 5100 + rank)}), device=device, dtype=torch.long)
    ci = torch.tensor(sorted({0, cn - 1, *np_sample(cn, 62, 5200 + rank)}), device=device, dtype=torch.long)
    ex_r = a_all[ri].double() @ b.double()
    ex_c = a_all.double() @ b[:, ci].double()
    er, ec_ = error_metrics(torch, c[ri], ex_r), error_metrics(torch, c[:, ci], ex_c)
    t = torch.tensor([max(er[q], ec_[q]) for q in ("max_rel", "fro_rel", "max_abs")], device=device, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    rows_cols = dict(zip(("max_rel", "fro_rel", "max_abs"), t.tolist()))
    rows_cols["how"] = "64 seeded rows and 64 seeded columns of every rank's block against GPU FP64 products; maxima over ranks"
    del a_all, c_chk, ex_r, ex_c

    # ---- correctness of every rank's block: sampled rows against the FP64 host loop (outside the timed region)
    rows = [0, 1, m // 2 - 1, m // 2, m - 1]
    a_rows = a[rows].contiguous() if rank == 0 else torch.empty((len(rows), k), device=device)
    dist.broadcast(a_rows, src=0)
    dmax, rmax, d32, nonfinite = sampled_accuracy(torch, np, cpu, a_rows.cpu().numpy(), b, c[rows])
    t = torch.tensor([dmax, rmax, d32, nonfinite], device=device, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dmax, rmax, d32, nonfinite = t.tolist()
    accuracy = {"rows_checked_per_rank": len(rows), "ranks_checked": world, "max_rel": dmax / rmax,
                "fp32_fma_max_rel": d32 / rmax, "nonfinite_fraction": nonfinite,
                "how": "each rank: sampled rows of its C block against the FP64 host loop; maxima over all ranks",
                "rows_and_columns_vs_gpu_fp64": rows_cols}

    # ---- end to end at N GPUs: every rank's B block (and A on rank 0) start in pinned host memory on the
    #      rank's NUMA node, every rank's C block ends there; copy-in, broadcast, GEMM and copy-out pipelined
    cpus = bind_to_gpu_numa_node(device.index)
    bh = torch.empty((k, cn), dtype=torch.float32, pin_memory=True)
    ch = torch.empty((m, cn), dtype=torch.float32, pin_memory=True)
    bh.copy_(b)
    ah = None
    if rank == 0:
        ah = torch.empty((m, k), dtype=torch.float32, pin_memory=True)
        ah.copy_(a)
    torch.cuda.synchronize()

    def e2e_step():
        tcec.sgemm_column_shard_host(ah, bh, ch, m, k, root=0, policy=policy, panel_rows=args.panel_rows)

    e2e_step()
    torch.cuda.synchronize()
    same = torch.tensor([1.0 if torch.equal(ch[-256:], c[-256:].cpu()) else 0.0], device=device, dtype=torch.float64)
    dist.all_reduce(same, op=dist.ReduceOp.MIN)
    e2e_steps = max(2, min(args.steps, 3))
    ms_e = max_over_ranks(torch, time_loop(torch, e2e_step, e2e_steps, True), device, True) / e2e_steps
    # what the host allows: every rank copies its C block out at the same time and nothing else runs
    ms_d2h = max_over_ranks(torch, time_loop(torch, lambda: ch.copy_(c, non_blocking=True), 1, True), device, True)
    e2e = {"value": flop / (ms_e * 1e-3) * 1e-12, "unit": UNIT,
           "h2d_bytes_per_step": 4 * (m * k + k * n), "d2h_bytes_per_step": 4 * m * n, "ms_per_step": ms_e,
           "copy_out_alone_ms": ms_d2h,
           "copy_out_alone_is": f"all {world} ranks copying their C blocks to pinned host memory at once, nothing else "
                                f"running: {4.0 * m * n / world / (ms_d2h * 1e-3) * 1e-9:.1f} GB/s per rank",
           "matches_device_resident_result": bool(same.item() == 1.0), "numa_cpus_per_rank": cpus,
           "how": "tcec_sgemm_column_shard_host on every rank: pinned host B block in, C block out, A from pinned host "
                  "memory on rank 0; copy-in, split, broadcast, GEMM and copy-out pipelined in row panels on four streams"}
    del bh, ch, ah
    tcec.device_status()
    del a, b, c

    batched = batched_extra(torch, tcec, sharded, peaks, args, rank, world, device, True)
    if rank == 0:
        peak = peaks["bf16_burst"] / 3.0
        line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
                "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True,
                "scaling": "strong", "vs_baseline": None, "dtype": "f16 hi/lo products, f32 accumulate",
                "data": "synthetic", "config": bench_config(world, args.size, (m, n, k), args.panel_rows),
                "clocks": clocks,
                # rank 0 per step: split of B, one split per row panel of A, the GEMM launch and its helper launch
                "gpu_launches": (1 + panels + 2) * args.steps,
                "roofline": {"bound": "tensor", "achieved": value / world, "peak": peak, "unit": UNIT,
                             "frac": value / world / peak, "traffic": None,
                             "peak_is": f"per GPU: dense 16-bit tensor peak (burst) / 3 products, {peaks['source']}",
                             "frac_of_sustained_peak": value / world / (peaks["bf16_sustained"] / 3.0),
                             "kernel": "tcec_gemm_panels_kernel<256,fp16,ec>, one persistent launch per GPU and step"},
                "accuracy": accuracy, "communication": comm, "e2e": e2e, "batched_256": batched}
        line["config"]["promote_k"] = tcec.get_option("promote_k")
        line["config"]["comm_sms"] = tcec.get_option("comm_sms")
        print(json.dumps(line), flush=True)
    tcec.comm_destroy()
    dist.destroy_process_group()


def run_ours(args):
    import numpy as np
    import torch

    from wmma_extension_b200 import sharded, tcec

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device; there is no CPU path (use --impl reference)")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    tcec.load()
    peaks = measured_peaks()
    if world > 1:
        import datetime

        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=device, timeout=datetime.timedelta(seconds=300))
        run_sharded(args, torch, np, tcec, sharded, peaks, device, rank, world)
    else:
        run_single(args, torch, np, tcec, sharded, peaks, device)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--size", type=int, default=16384, help="M = N = K of the one-GPU workload")
    ap.add_argument("--large", type=int, nargs=3, default=list(LARGE), metavar=("M", "N", "K"),
                    help="shape of the column-sharded workload")
    ap.add_argument("--panel-rows", type=int, default=2048)
    ap.add_argument("--policy", default="fp16_ec", choices=["fp16_ec", "tf32_ec", "fp16_no_ec", "tf32_no_ec"],
                    help="with --only kernel: the policy of the GEMM")
    ap.add_argument("--batched", type=int, default=8192, help="matrices of the batched 256^3 configuration")
    ap.add_argument("--only", default="", choices=["", "kernel", "batched"],
                    help="kernel: nothing but the headline GEMM of one GPU; batched: nothing but the batched "
                         "configuration (the commands of the profiler captures)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
