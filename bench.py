"""Benchmark of the k-means iteration hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c2] [--impl reference]

A step is one Lloyd iteration (assignment + update + divide) over the whole workload.  The
default workload is the headline configuration "c2": N = 2^21 points, dim 32, k 1024, fp32,
SoA points, i.i.d. uniform [0,1) coordinates, initial means = the first k points (seeded
synthetic data; the reference measures on its own random generator, no dataset is involved).
With N GPUs (one process per GPU, torchrun) every rank holds its own 2^21-point shard of a
G * 2^21 point data set (weak scaling) and the k x dim sums and k sizes are exchanged between
the ranks every iteration.  `--workload c5 --scaling strong` runs the sharded 2^28-point
configuration as the headline instead.

Rank 0 prints ONE JSON line: `value` is giga distance evaluations per second (N_total * k /
iteration time) with the data resident in HBM, timed with CUDA events on the launching stream
and maximised over ranks; `e2e` is the same metric through the host-buffer C-ABI calls with
the host<->device copies inside the timed region; `roofline` describes the dominant kernel
(the assignment) against a TF32 matrix-multiply rate measured in the same run; `cpu_baseline`
is the reference's serial CPU k-means on a bounded sample; `parity` is a check of one more
iteration against the CPU oracle and across ranks (outside the timed region); `c5_strong` is
the sharded 2^28-point configuration at the same number of GPUs, and `configs` (one GPU only)
holds the remaining benchmark configurations.  `--no-extras` skips those extra measurements.

`--impl reference` times the reference's own serial CPU implementation instead (compiled from
its headers into oracle/_ref, else the plain-C port in oracle/).
"""
import argparse
import hashlib
import json
import os
import statistics
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

V100_PUBLISHED_GEVALS = 84.4  # reference's best variant, N=2M d=32 k=1024, V100 (results/README.md:20)
# DRAM bytes (read + write, from one profiler capture) that one assignment launch on workload c2
# moves per point: the capture ran on 2^19 points (138.81 MB read + 6.79 MB written); the traffic is
# the point operands, read once, so it grows in proportion to the points.
C2_ASSIGN_TC_DRAM_BYTES_PER_POINT = (138.81e6 + 6.79e6) / (1 << 19)
# the same for the one-CTA tensor-core kernel on c5's shape (2^24-point capture: 2.215 GB read, 67.8 MB written)
# and for the CUDA-core kernel on c3's shape (2^22-point capture: 33.6 MB read; the 16.8 MB of assignments
# stayed in L2 at that size and are counted as written)
C5_ASSIGN_TC_DRAM_BYTES_PER_POINT = (2.215e9 + 67.8e6) / (1 << 24)
C3_ASSIGN_SIMT_DRAM_BYTES_PER_POINT = (33.6e6 + 16.8e6) / (1 << 22)
PARITY_SAMPLE = 4096
PHASE_STEPS = 8     # instrumented iterations behind the timed ones, for `phases_ms`


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="c2")
    ap.add_argument("--scaling", default=None, choices=[None, "weak", "strong"])
    ap.add_argument("--n", type=int, default=None, help="override the number of points (per job)")
    ap.add_argument("--assign", default="auto", choices=["auto", "exact", "simt", "tc"])
    ap.add_argument("--update", default="auto", choices=["auto", "shared", "global", "rows", "sorted"])
    ap.add_argument("--no-fuse", action="store_true",
                    help="keep the update a launch of its own where the assignment kernel could accumulate the sums")
    ap.add_argument("--fuse-all", action="store_true",
                    help="let the assignment kernel accumulate the sums wherever it can, also where the library's default keeps two passes")
    ap.add_argument("--exchange", default="auto", choices=["auto", "nccl", "peer"],
                    help="how the ranks exchange sums and sizes: NCCL all-reduce, or the library's peer-load kernel")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="skip the c5 strong-scaling run and the other configurations")
    ap.add_argument("--no-parity", action="store_true")
    ap.add_argument("--seed", type=int, default=42)
    return ap.parse_args()


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return dict(hbm_gbs=p["hbm_gbs"], bf16_tflops=p["bf16_tflops"],
                    bf16_tflops_sustained=p.get("bf16_tflops_sustained"), source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, source="fallback")


def measure_tf32_peak(torch, size=8192, reps=10):
    """Dense TF32 matrix-multiply rate of this GPU right now (TFLOP/s): a library GEMM with TF32
    allowed, best of `reps` - a measurement only, the denominator of the tensor roofline."""
    old = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = True
    try:
        a = torch.randn(size, size, device="cuda", dtype=torch.float32)
        b = torch.randn(size, size, device="cuda", dtype=torch.float32)
        for _ in range(3):
            torch.matmul(a, b)
        best = float("inf")
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for _ in range(reps):
            e0.record()
            torch.matmul(a, b)
            e1.record()
            e1.synchronize()
            best = min(best, e0.elapsed_time(e1))
        del a, b
        return 2.0 * size ** 3 / (best * 1e-3) / 1e12
    finally:
        torch.backends.cuda.matmul.allow_tf32 = old


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons through NVML (read-only) while a region runs."""

    def __init__(self, index):
        super().__init__(daemon=True)
        self.index = index
        self.samples = []
        self.reasons = set()
        self.max_mhz = None
        self._stop_evt = threading.Event()
        self.ok = False
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
            self.ok = True
        except Exception:
            self.ok = False

    def run(self):
        if not self.ok:
            return
        nv = self.nv
        names = {
            "hw_slowdown": getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8),
            "hw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40),
            "sw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20),
            "sw_power_cap": getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4),
            "hw_power_brake": getattr(nv, "nvmlClocksEventReasonHwPowerBrakeSlowdown", 0x80),
        }
        while not self._stop_evt.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                try:
                    mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for k, bit in names.items():
                    if mask & bit:
                        self.reasons.add(k)
            except Exception:
                pass
            time.sleep(0.005)

    def stop(self):
        self._stop_evt.set()
        self.join(timeout=2)
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None,
                "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(self.samples)}


def physical_gpu_index(local_index):
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        parts = [p for p in vis.split(",") if p.strip() != ""]
        try:
            return int(parts[local_index])
        except Exception:
            return local_index
    return local_index


def device_rows(torch, workloads, spec, n_total, begin, count, seed, chunk=1 << 22):
    """Rows [begin, begin+count) of a large workload generated on the GPU in chunks seeded by
    (seed, chunk index), so that every rank count sees the same global data set.  Returns the flat
    device tensor in the workload's layout and the first k rows (initial means) as a numpy array."""
    k, dim, lay = spec["k"], spec["dim"], spec["layout"]
    kind, sigma = spec["kind"], spec.get("sigma", 0.05)
    out = torch.empty(count * dim, dtype=torch.float32, device="cuda")
    view = out.view(count, dim) if lay == 0 else out.view(dim, count)
    centres = torch.from_numpy(workloads.mixture_centres(k, dim, seed)).cuda() if kind == "mixture" else None
    weights = torch.from_numpy(workloads.mixture_weights(k, spec.get("zipf"))).float().cuda() if kind == "mixture" else None
    gen = torch.Generator(device="cuda")

    def block(c):
        c0, c1 = c * chunk, min(n_total, (c + 1) * chunk)
        gen.manual_seed(seed * 1000003 + c)
        if kind == "uniform":
            return torch.rand((c1 - c0, dim), generator=gen, device="cuda")
        if kind == "mixture":
            which = torch.multinomial(weights, c1 - c0, replacement=True, generator=gen)
            return centres[which] + sigma * torch.randn((c1 - c0, dim), generator=gen, device="cuda")
        x = torch.randn((c1 - c0, dim), generator=gen, device="cuda")
        return x / x.norm(dim=1, keepdim=True)

    for c in range(begin // chunk, (begin + count - 1) // chunk + 1):
        c0 = c * chunk
        rows = block(c)
        lo, hi = max(begin, c0), min(begin + count, c0 + rows.shape[0])
        part = rows[lo - c0:hi - c0]
        if lay == 0:
            view[lo - begin:hi - begin] = part
        else:
            view[:, lo - begin:hi - begin] = part.t()
        del rows, part
    first = block(0)[:k].cpu().numpy()
    return out, first


def cpu_reference_leg(workloads, spec, seed, sample_n, steps, warmup):
    """Times the reference's serial CPU k-means, one iteration per step, on the first
    `sample_n` points of the workload (same k, dim, layouts, initial means)."""
    import oracle
    ref = oracle.ref()
    kind = "reference" if ref is not None else "port"
    k, dim, lay, laym = spec["k"], spec["dim"], spec["layout"], spec["layout_means"]
    rows = workloads.generate_rows(spec["kind"], sample_n, dim, k, seed, spec.get("sigma", 0.05), spec.get("zipf"))
    data, means = workloads.to_layout(rows, lay), workloads.to_layout(rows[:k], laym)

    def one(m):
        if ref is not None:
            return ref.kmeans(data, m, sample_n, k, dim, 1, lay, laym)[0]
        return oracle.kmeans(data, m, sample_n, k, dim, 1, lay, laym)[0]

    m = means
    for _ in range(warmup):
        m = one(m)
    t0 = time.perf_counter()
    for _ in range(steps):
        m = one(m)
    dt = (time.perf_counter() - t0) / max(1, steps)
    return dict(value=sample_n * k / dt / 1e9, unit="G dist-evals/s", cores=1, kind=kind,
                sample="first %d points of the workload (same k, dim, layout), %d iteration(s), %.2f s each; "
                       "serial by construction (1 thread)" % (sample_n, steps, dt)), dt


class Job:
    """One workload resident on this rank's GPU behind a k-means handle."""

    def __init__(self, ctx, name, scaling, n_override=None, host_copy=False):
        torch, pkg, workloads, args = ctx["torch"], ctx["pkg"], ctx["workloads"], ctx["args"]
        world, rank = ctx["world"], ctx["rank"]
        spec = dict(workloads.CONFIGS[name])
        spec["layout_means"] = spec["layout"]
        if n_override:
            spec["n"] = n_override
        self.spec, self.name, self.scaling = spec, name, scaling
        k, dim, lay, laym = spec["k"], spec["dim"], spec["layout"], spec["layout_means"]
        self.n_total = spec["n"] * world if scaling == "weak" else spec["n"]
        self.begin, self.count = pkg.shard_range(self.n_total, world, rank)
        self.host_points = None
        if host_copy and self.count * dim * 4 <= (2 << 30):
            rows = workloads.generate_rows(spec["kind"], self.n_total, dim, k, args.seed, spec.get("sigma", 0.05),
                                           spec.get("zipf"), begin=self.begin, count=self.count)
            first = rows[:k] if self.begin == 0 else workloads.generate_rows(
                spec["kind"], self.n_total, dim, k, args.seed, spec.get("sigma", 0.05), spec.get("zipf"), begin=0, count=k)
            self.host_points = torch.from_numpy(workloads.to_layout(rows, lay)).pin_memory()
            del rows
            self.dev_points = self.host_points.to("cuda", non_blocking=False)
        else:
            self.dev_points, first = device_rows(torch, workloads, spec, self.n_total, self.begin, self.count, args.seed)
        self.host_means = torch.from_numpy(workloads.to_layout(first, laym)).pin_memory()
        self.dev_means = self.host_means.to("cuda")
        self.km = None

    def handle(self, ctx, va=0, vu=0, device_init=True, fuse=True):
        torch, pkg, args = ctx["torch"], ctx["pkg"], ctx["args"]
        spec = self.spec
        km = pkg.KMeans(layout=spec["layout"], layout_means=spec["layout_means"], device=ctx["local_rank"],
                        variant_assign=va, variant_update=vu)
        km.set_stream(ctx["stream"].cuda_stream)
        if device_init:
            km.initialize_device(spec["dim"], spec["k"], self.count, 1, self.dev_points.data_ptr(), self.dev_means.data_ptr())
        else:
            km.initialize(spec["dim"], spec["k"], self.count, 1, self.host_points.numpy(), self.host_means.numpy())
        if not fuse:
            km.set_option("fuse_update", 0)
        elif args.fuse_all:
            km.set_option("fuse_update", 2)
        if ctx["world"] > 1:
            ctx["join"](km)
        return km

    def rows_sample(self, torch, idx):
        """(len(idx), dim) numpy rows of this rank's shard."""
        spec = self.spec
        ti = torch.from_numpy(idx.astype(np.int64)).cuda()
        view = self.dev_points.view(self.count, spec["dim"]) if spec["layout"] == 0 else self.dev_points.view(spec["dim"], self.count).t()
        return view[ti].contiguous().cpu().numpy()


def timed_run(ctx, km, steps, warmup, sample_clocks=True):
    """`warmup` untimed iterations, then exactly `steps` timed with CUDA events on the launching
    stream between two barriers; returns (ms per step maximised over ranks, clocks, phases, counters)."""
    torch, dist, stream = ctx["torch"], ctx["dist"], ctx["stream"]

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    # The ranks leave a host-side barrier up to milliseconds apart (more so with eight processes on
    # shared cores), and the rank that is first would count that lead as waiting time in its first
    # exchange.  So the last warm-up step is enqueued behind the barrier, directly in front of the
    # timed steps: its exchange lines the ranks' streams up, and the events bracket exactly `steps`
    # iterations that all GPUs start together.
    # The timed steps run without the library's per-phase events (six records per iteration cost 2-5 %);
    # the phase times come from PHASE_STEPS instrumented iterations behind them.
    km.set_option("phase_timing", 0)
    km.run(max(warmup - 1, 0))
    barrier()
    sampler = ClockSampler(physical_gpu_index(ctx["local_rank"])) if sample_clocks else None
    if sampler:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if warmup > 0:
        km.run_async(1)
    e0.record(stream)
    t_host = time.perf_counter()
    km.run_async(steps)
    enqueue_ms = (time.perf_counter() - t_host) * 1e3
    e1.record(stream)
    barrier()
    km.synchronize()
    clocks = sampler.stop() if sampler else None
    ms_total = e0.elapsed_time(e1)
    km.set_option("phase_timing", 1)
    km.run(PHASE_STEPS + 1)     # the library records the last PHASE_STEPS; the one in front lines the ranks up again
    barrier()
    phases = km.phase_ms()
    counters = km.counters()
    by_rank = None
    if dist is not None:
        t = torch.tensor([ms_total], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_total = float(t.item())
        # per-rank phase times (each on its own device clock): the spread of the work before the
        # exchange is rank skew, the smallest exchange time is what the exchange itself costs
        names = ["assign", "recheck", "update", "allreduce", "finalize", "iteration"]
        mine = torch.tensor([phases[x] for x in names], device="cuda", dtype=torch.float64)
        allp = [torch.zeros_like(mine) for _ in range(ctx["world"])]
        dist.all_gather(allp, mine)
        allp = torch.stack(allp).cpu().numpy()
        before = allp[:, 0] + allp[:, 1] + allp[:, 2]
        t2 = torch.tensor([enqueue_ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t2, op=dist.ReduceOp.MAX)
        by_rank = {"host_enqueue_ms_per_step_max": float(t2.item()) / steps,
                   "compute_before_exchange_min": float(before.min()), "compute_before_exchange_max": float(before.max()),
                   "exchange_min": float(allp[:, 3].min()), "exchange_max": float(allp[:, 3].max()),
                   "finalize_max": float(allp[:, 4].max()), "iteration_max": float(allp[:, 5].max())}
    return ms_total / steps, clocks, phases, counters, by_rank


def parity_check(ctx, job, km):
    """One more iteration, outside any timed region, checked against the CPU oracle and across the
    ranks: a sample of this rank's assignment bit for bit against serial.hpp's arg-min (restated in
    oracle/) for the means the iteration started from, the sizes adding up to the number of points,
    size-weighted means adding up to the sum of all points, and identical means on every rank."""
    import oracle
    torch, dist = ctx["torch"], ctx["dist"]
    spec = job.spec
    k, dim, lay, laym = spec["k"], spec["dim"], spec["layout"], spec["layout_means"]
    prev = km.getMeans()
    km.run(1)
    means, sizes = km.getMeans(), km.getSizes()
    rng = np.random.default_rng(1234 + ctx["rank"])
    m = min(PARITY_SAMPLE if dim <= 64 else 1024, job.count)
    idx = np.sort(rng.choice(job.count, m, replace=False))
    rows = job.rows_sample(torch, idx)
    got = km.getAssignment()[idx]
    want = oracle.assign(ctx["workloads"].to_layout(rows, lay), prev, m, k, dim, lay, laym, threads=8)
    mismatches = int((got != want).sum())
    # conservation: sum_c size_c * mean_c == sum of all points, per dimension (double precision)
    view = job.dev_points.view(job.count, dim) if lay == 0 else job.dev_points.view(dim, job.count).t()
    total = view.sum(dim=0, dtype=torch.float64)
    abs_total = torch.linalg.vector_norm(view, ord=1, dim=0, dtype=torch.float64)    # sum of |x| per dimension: the error scale
    size_sum = int(sizes.astype(np.int64).sum())
    digest = int.from_bytes(hashlib.sha256(means.tobytes()).digest()[:7], "little")
    same_means = True
    if dist is not None:
        dist.all_reduce(total)
        dist.all_reduce(abs_total)
        d = torch.tensor([digest], device="cuda", dtype=torch.int64)
        alld = [torch.zeros_like(d) for _ in range(ctx["world"])]
        dist.all_gather(alld, d)
        same_means = len({int(x.item()) for x in alld}) == 1
        mm = torch.tensor([mismatches], device="cuda", dtype=torch.int64)
        dist.all_reduce(mm)
        mismatches = int(mm.item())
    mrows = ctx["workloads"].from_layout(means, k, dim, laym).astype(np.float64)
    got_total = (mrows * sizes.astype(np.float64)[:, None]).sum(axis=0)
    want_total = total.cpu().numpy()
    scale = max(float(abs_total.max().item()), 1e-30)
    cons_err = float(np.abs(got_total - want_total).max() / scale)
    ok = mismatches == 0 and size_sum == job.n_total and same_means and cons_err <= 1e-5
    return {"ok": bool(ok), "sampled_points_per_rank": int(m), "assignment_mismatches_vs_oracle": mismatches,
            "sizes_sum": size_sum, "n_total": int(job.n_total), "means_identical_on_all_ranks": bool(same_means),
            "conservation_rel_err": cons_err,
            "what": "one extra iteration: sampled assignment == oracle arg-min for the previous means (bit-exact), "
                    "sum of sizes == N_total, sum_c size_c*mean_c == sum of points (<= 1e-5), means hash equal on all ranks"}


def roofline_of(ctx, job, phases, counters, plan, ms_step, tf32_peak):
    peaks = ctx["peaks"]
    spec = job.spec
    k, dim = spec["k"], spec["dim"]
    flops_iter = 2.0 * job.count * k * dim            # algorithmic flops of one assignment launch on this rank
    bytes_iter = 4.0 * job.count * dim
    assign_ms = phases["assign"]
    roofline = None
    if assign_ms > 0:
        if counters["assign_variant"] == "tc":
            ach = flops_iter / (assign_ms * 1e-3) / 1e12
            traffic = None
            if job.name == "c2" and plan["kernel"] == "tc_pair":
                traffic = C2_ASSIGN_TC_DRAM_BYTES_PER_POINT * job.count
            elif job.name == "c5" and plan["kernel"] == "tc_resident":
                traffic = C5_ASSIGN_TC_DRAM_BYTES_PER_POINT * job.count
            ksteps = (min(dim, 32) + 7) // 8 if dim <= 32 else None
            issued = (3.0 * ksteps + 1.0) / ksteps if ksteps else 3.0 + 8.0 / dim
            roofline = {"bound": "tensor", "achieved": ach, "peak": tf32_peak, "unit": "TFLOP/s", "frac": ach / tf32_peak,
                        "peak_tf32_measured": tf32_peak,
                        "frac_tensor_issued": issued * ach / tf32_peak,
                        "tensor_flops_per_algorithmic_flop": issued,
                        "frac_vs_half_bf16_burst": ach / (peaks["bf16_tflops"] * 0.5),
                        "traffic": traffic,
                        "traffic_unit": "bytes per launch (profiler DRAM read+write per point of a reduced-size capture x points of this launch)",
                        "kernel": "assignment (%s)" % plan["kernel"], "kernel_ms": assign_ms,
                        "peak_note": "peak = TF32 library GEMM (8192^3, best of 10) measured in this run; `frac` counts "
                                     "algorithmic flops 2*N*k*d; the split-TF32 scheme issues `tensor_flops_per_algorithmic_flop` "
                                     "tensor flops for each, `frac_tensor_issued` is that work against the same peak; half the %s "
                                     "bf16 burst peak is %.1f TFLOP/s" % (peaks["source"], peaks["bf16_tflops"] * 0.5)}
        else:
            ach = bytes_iter / (assign_ms * 1e-3) / 1e9
            roofline = {"bound": "hbm", "achieved": ach, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                        "frac": ach / peaks["hbm_gbs"],
                        "traffic": C3_ASSIGN_SIMT_DRAM_BYTES_PER_POINT * job.count if job.name == "c3" else None,
                        "traffic_unit": "bytes per launch (profiler DRAM read+write per point of a reduced-size capture x points of this launch)",
                        "kernel": "assignment (%s)" % plan["kernel"], "kernel_ms": assign_ms,
                        "peak_note": "%s HBM copy bandwidth; algorithmic bytes 4*N*d" % peaks["source"]}
    # the contractual whole-iteration roofline: slower of 2Nkd flops at the TF32 rate and 4Nd bytes at HBM bandwidth
    t_roof = max(flops_iter / (tf32_peak * 1e12), bytes_iter / (peaks["hbm_gbs"] * 1e9))
    iteration_roofline = {"roofline_ms": t_roof * 1e3, "frac": t_roof * 1e3 / ms_step,
                          "peaks": "tf32 = %.1f TFLOP/s (measured in this run), hbm = %.1f GB/s (%s)" % (
                              tf32_peak, peaks["hbm_gbs"], peaks["source"])}
    return roofline, iteration_roofline


def extra_config(ctx, name, scaling, steps, warmup, tf32_peak):
    """One more configuration measured after the headline one (device-generated data)."""
    torch = ctx["torch"]
    job = Job(ctx, name, scaling)
    km = job.handle(ctx)
    ms_step, clocks, phases, counters, by_rank = timed_run(ctx, km, steps, warmup, sample_clocks=True)
    plan = km.assign_plan()
    roofline, iteration_roofline = roofline_of(ctx, job, phases, counters, plan, ms_step, tf32_peak)
    parity = None if ctx["args"].no_parity else parity_check(ctx, job, km)
    spec = job.spec
    out = {"workload": "%s: N_total=%d (%d on this rank) x dim %d, k=%d, fp32, %s points, %s" % (
        name, job.n_total, job.count, spec["dim"], spec["k"], "SoA" if spec["layout"] == 1 else "AoS", spec["kind"]),
        "scaling": scaling, "steps": steps, "warmup": warmup, "ms_per_step": ms_step,
        "value": job.n_total * spec["k"] / (ms_step * 1e-3) / 1e9, "unit": "G dist-evals/s",
        "phases_ms": phases, "phases_ms_across_ranks": by_rank, "variants": counters, "plan": plan, "clocks": clocks,
        "roofline": roofline, "iteration_roofline": iteration_roofline, "parity": parity,
        "gpu_launches": counters["launches_per_iter"] * steps}
    km.cleanup()
    del job, km
    torch.cuda.empty_cache()
    return out


def main():
    args = parse_args()
    import __graft_entry__ as entry
    pkg = entry.load()
    import importlib
    workloads = importlib.import_module("cuda_kmeans_b200.workloads")

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    spec = dict(workloads.CONFIGS[args.workload])
    spec["layout_means"] = spec["layout"]
    if args.n:
        spec["n"] = args.n
    k, dim, lay, laym = spec["k"], spec["dim"], spec["layout"], spec["layout_means"]
    scaling = args.scaling or ("strong" if args.workload == "c5" else "weak")
    n_total_cfg = spec["n"] * args.gpus if scaling == "weak" else spec["n"]
    per_gpu = " per GPU, N_total=%d" % n_total_cfg if scaling == "weak" else " in total, sharded over the GPUs"
    config = {"workload": "%s: N=%d%s x dim %d, k=%d, fp32, %s points" % (
        args.workload, spec["n"], per_gpu, dim, k, "SoA" if lay == 1 else "AoS"),
        "distribution": spec["kind"], "init": "first k points", "l2": "inputs exceed L2 (no flush needed)"
        if spec["n"] * dim * 4 > 126e6 else "inputs fit L2: working set is re-read from L2 between steps",
        "timing": "CUDA events on the launching stream around exactly `steps` iterations, max over ranks; W-1 warm-up steps, "
                  "barrier + synchronize, then the last warm-up step and the timed steps are enqueued back to back (the "
                  "exchange of that step lines the GPUs up, so the ranks' different exits from the barrier are not timed)"}

    # ---------------- reference arm: the reference's CPU implementation ----------------
    if args.impl == "reference":
        if rank != 0:
            return 0
        # bounded sample: about 60 s of serial CPU work for the whole run, at least k points
        budget_evals = 60.0 * 0.012e9 * (32.0 / max(dim, 1)) / max(1, args.steps + min(args.warmup, 1))
        sample_n = 1 << max(0, int(np.floor(np.log2(max(1.0, budget_evals / k)))))
        sample_n = int(min(spec["n"], max(sample_n, 1 << int(np.ceil(np.log2(k))), 256)))
        base, dt = cpu_reference_leg(workloads, spec, args.seed, sample_n, args.steps, min(args.warmup, 1))
        line = {"metric": "k-means iteration throughput", "value": base["value"], "unit": "G dist-evals/s",
                "n_gpus": args.gpus, "steps": args.steps, "warmup": min(args.warmup, 1), "ms_per_step": dt * 1e3,
                "higher_is_better": True, "scaling": scaling, "vs_baseline": None, "dtype": "f32",
                "data": "synthetic", "impl": "reference", "config": config, "cpu_baseline": base,
                "e2e": {"value": base["value"], "unit": "G dist-evals/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                "gpu_launches": 0,
                "note": "each step is one iteration on a bounded sample; ms_per_step is for the sample, "
                        "value (dist-evals/s) is size-independent"}
        print(json.dumps(line))
        return 0

    # ---------------- B200 arm ----------------
    import torch
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback)")
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group(backend="nccl", device_id=torch.device("cuda", local_rank))

    stream = torch.cuda.Stream()
    torch.cuda.set_stream(stream)
    exchange_used = {"mode": "none"}

    def join(km):
        """Makes `km` one rank of the job: NCCL communicator through the launcher's process group, then
        (unless --exchange nccl) the peer-memory exchange."""
        uid = torch.zeros(128, dtype=torch.uint8, device="cuda")
        if rank == 0:
            uid.copy_(torch.frombuffer(bytearray(pkg.comm_unique_id()), dtype=torch.uint8))
        dist.broadcast(uid, 0)
        km.comm_init(bytes(uid.cpu().numpy().tobytes()), world, rank)
        exchange_used["mode"] = "nccl"
        if args.exchange != "nccl" and hasattr(km, "peer_exchange_init"):
            if km.peer_exchange_init(dist, torch):
                exchange_used["mode"] = "peer"
            elif args.exchange == "peer":
                raise SystemExit("--exchange peer: the peer-memory exchange could not be set up")

    ctx = dict(torch=torch, pkg=pkg, workloads=workloads, args=args, world=world, rank=rank, local_rank=local_rank,
               dist=dist, stream=stream, join=join, peaks=measured_peaks())

    tf32_peak = measure_tf32_peak(torch)
    if dist is not None:
        t = torch.tensor([tf32_peak], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        tf32_peak = float(t.item())

    va = {"auto": 0, "exact": 1, "simt": 2, "tc": 3}[args.assign]
    vu = {"auto": 0, "shared": 1, "global": 2, "rows": 3, "sorted": 5}[args.update]
    job = Job(ctx, args.workload, scaling, n_override=args.n, host_copy=True)
    n_total, count = job.n_total, job.count
    km = job.handle(ctx, va, vu, fuse=not args.no_fuse)
    ms_step, clocks, phases, counters, by_rank = timed_run(ctx, km, args.steps, args.warmup)
    value = n_total * k / (ms_step * 1e-3) / 1e9
    plan = km.assign_plan()
    parity = None if args.no_parity else parity_check(ctx, job, km)

    # ---------------- end to end through the host-buffer calls ----------------
    e2e = None
    if not args.no_e2e and job.host_points is not None:
        e2e_steps = max(3, min(args.steps, 20))
        km2 = job.handle(ctx, va, vu, device_init=False, fuse=not args.no_fuse)
        hp, hm = job.host_points.numpy(), job.host_means.numpy()
        out_means = torch.empty(k * dim, dtype=torch.float32).pin_memory()
        out_asg = torch.empty(count, dtype=torch.int32).pin_memory()

        def barrier():
            if dist is not None:
                dist.barrier()
            torch.cuda.synchronize()

        def e2e_step():
            # host -> device copy of points and means, preprocessing, one iteration, results back
            pkg.check(pkg.lib().bkm_initialize(km2._h, hp.ctypes.data, hm.ctypes.data))
            pkg.check(pkg.lib().bkm_run(km2._h, 1))
            pkg.check(pkg.lib().bkm_get_means(km2._h, out_means.data_ptr()))
            pkg.check(pkg.lib().bkm_get_assignment(km2._h, out_asg.data_ptr()))

        for _ in range(3):
            e2e_step()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        e0.record(stream)
        for _ in range(e2e_steps):
            e2e_step()
        e1.record(stream)
        barrier()
        wall = (time.perf_counter() - t0) * 1e3 / e2e_steps
        # the host calls are synchronous: take the larger of device-event and host wall time
        ms_e2e = max(e0.elapsed_time(e1) / e2e_steps, wall)
        if dist is not None:
            t = torch.tensor([ms_e2e], device="cuda", dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms_e2e = float(t.item())
        e2e = {"value": n_total * k / (ms_e2e * 1e-3) / 1e9, "unit": "G dist-evals/s",
               "h2d_bytes_per_step": int(count * dim * 4 + k * dim * 4),
               "d2h_bytes_per_step": int(k * dim * 4 + count * 4),
               "ms_per_step": ms_e2e, "wall_ms_per_step": wall, "steps": e2e_steps,
               "call": "bkm_initialize(host) + bkm_run(1) + bkm_get_means + bkm_get_assignment, pinned host buffers"}
        km2.cleanup()

    roofline, iteration_roofline = roofline_of(ctx, job, phases, counters, plan, ms_step, tf32_peak)

    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        sample_n = min(spec["n"], max(1 << 12, (1 << 26) // (k * max(1, dim // 32 + (dim % 32 > 0)))))
        cpu_baseline, _ = cpu_reference_leg(workloads, spec, args.seed, sample_n, 1, 0)

    km.cleanup()
    del km, job
    torch.cuda.empty_cache()

    # ---------------- the other configurations (outside the headline measurement) ----------------
    c5_strong, configs = None, None
    if not args.no_extras and args.workload == "c2" and not args.n:
        c5_strong = extra_config(ctx, "c5", "strong", 10, 3, tf32_peak)
        if world == 1:
            configs = {"c1": extra_config(ctx, "c1", "strong", 200, 20, tf32_peak),
                       "c3": extra_config(ctx, "c3", "strong", 50, 5, tf32_peak),
                       "c4": extra_config(ctx, "c4", "strong", 10, 3, tf32_peak)}

    if rank == 0:
        line = {"metric": "k-means iteration throughput", "value": value, "unit": "G dist-evals/s",
                "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step,
                "higher_is_better": True, "scaling": scaling,
                "vs_baseline": value / V100_PUBLISHED_GEVALS if args.workload == "c2" else None,
                "vs_baseline_note": "reference's best published number for this shape: 25.45 ms = 84.4 G dist-evals/s on V100",
                "dtype": "f32", "data": "synthetic", "config": config, "e2e": e2e,
                "gpu_launches": counters["launches_per_iter"] * args.steps,
                "roofline": roofline, "iteration_roofline": iteration_roofline, "cpu_baseline": cpu_baseline,
                "clocks": clocks, "phases_ms": phases, "phases_ms_across_ranks": by_rank,
                "phases_from": "%d iterations with the library's per-phase CUDA events, directly behind the timed steps "
                               "(which run without them)" % PHASE_STEPS,
                "variants": counters, "plan": plan,
                "exchange": exchange_used["mode"], "parity": parity,
                "ns_per_input_float": ms_step * 1e6 / (n_total * dim),
                "c5_strong": c5_strong, "configs": configs}
        print(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
