"""Benchmark of the k-means iteration hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c2] [--impl reference]

A step is one Lloyd iteration (assignment + update + divide) over the whole workload.  The
default workload is the headline configuration "c2": N = 2^21 points, dim 32, k 1024, fp32,
SoA points, i.i.d. uniform [0,1) coordinates, initial means = the first k points (seeded
synthetic data; the reference measures on its own random generator, no dataset is involved).
With N GPUs (one process per GPU, torchrun) every rank holds its own 2^21-point shard of a
G * 2^21 point data set (weak scaling) and the k x dim sums and k sizes are all-reduced with
NCCL every iteration.  `--workload c5 --scaling strong` runs the sharded 2^28-point
configuration instead.

Rank 0 prints ONE JSON line: `value` is giga distance evaluations per second (N_total * k /
iteration time) with the data resident in HBM, timed with CUDA events on the launching stream
and maximised over ranks; `e2e` is the same metric through the host-buffer C-ABI calls with
the host<->device copies inside the timed region; `roofline` describes the dominant kernel
(the assignment); `cpu_baseline` is the reference's serial CPU k-means on a bounded sample.

`--impl reference` times the reference's own serial CPU implementation instead (compiled from
its headers into oracle/_ref, else the plain-C port in oracle/).
"""
import argparse
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
# dram__bytes_read.sum + dram__bytes_write.sum of one assign_tc_pair_kernel launch on workload c2: the ncu
# capture summarised in profiles/assign_tc_pair_kernel_c2.md was taken on a quarter of the points
# (138.88 MB + 4.71 MB); the traffic is the point operands, read once, so it scales with the points: x 4.
C2_ASSIGN_TC_DRAM_BYTES = 574.9e6


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
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
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
    config = {"workload": "%s: N=%d x dim %d, k=%d, fp32, %s points" % (
        args.workload, spec["n"], dim, k, "SoA" if lay == 1 else "AoS"),
        "distribution": spec["kind"], "init": "first k points", "l2": "inputs exceed L2 (no flush needed)"
        if spec["n"] * dim * 4 > 126e6 else "inputs fit L2: working set is re-read from L2 between steps"}

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

    n_total = spec["n"] * world if scaling == "weak" else spec["n"]
    begin, count = pkg.shard_range(n_total, world, rank)
    big = count * dim * 4 > (2 << 30)          # beyond 2 GiB the shard is generated on the device
    if big:
        dev_points, first = device_rows(torch, workloads, spec, n_total, begin, count, args.seed)
        host_points = None
        args.no_e2e = True                        # no host copy of a shard this large is kept
    else:
        rows = workloads.generate_rows(spec["kind"], n_total, dim, k, args.seed, spec.get("sigma", 0.05),
                                       spec.get("zipf"), begin=begin, count=count)
        first = rows[:k] if begin == 0 else workloads.generate_rows(
            spec["kind"], n_total, dim, k, args.seed, spec.get("sigma", 0.05), spec.get("zipf"), begin=0, count=k)
        host_points = torch.from_numpy(workloads.to_layout(rows, lay)).pin_memory()
        del rows
        dev_points = host_points.to("cuda", non_blocking=False)
    host_means = torch.from_numpy(workloads.to_layout(first, laym)).pin_memory()
    dev_means = host_means.to("cuda")

    va = {"auto": 0, "exact": 1, "simt": 2, "tc": 3}[args.assign]
    vu = {"auto": 0, "shared": 1, "global": 2, "rows": 3, "sorted": 5}[args.update]
    km = pkg.KMeans(layout=lay, layout_means=laym, device=local_rank, variant_assign=va, variant_update=vu)
    stream = torch.cuda.Stream()
    torch.cuda.set_stream(stream)
    km.set_stream(stream.cuda_stream)
    km.initialize_device(dim, k, count, args.steps, dev_points.data_ptr(), dev_means.data_ptr())
    if args.no_fuse:
        km.set_option("fuse_update", 0)
    if world > 1:
        uid = torch.zeros(128, dtype=torch.uint8, device="cuda")
        if rank == 0:
            uid.copy_(torch.frombuffer(bytearray(pkg.comm_unique_id()), dtype=torch.uint8))
        dist.broadcast(uid, 0)
        km.comm_init(bytes(uid.cpu().numpy().tobytes()), world, rank)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    km.run(args.warmup)
    barrier()
    sampler = ClockSampler(physical_gpu_index(local_rank))
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    km.run_async(args.steps)
    e1.record(stream)
    barrier()
    km.synchronize()
    clocks = sampler.stop()
    ms_total = e0.elapsed_time(e1)
    phases = km.phase_ms()
    counters = km.counters()
    if dist is not None:
        t = torch.tensor([ms_total], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_total = float(t.item())
    ms_step = ms_total / args.steps
    value = n_total * k / (ms_step * 1e-3) / 1e9

    # ---------------- end to end through the host-buffer calls ----------------
    e2e = None
    if not args.no_e2e and host_points is not None:
        e2e_steps = max(3, min(args.steps, 20))
        km2 = pkg.KMeans(layout=lay, layout_means=laym, device=local_rank, variant_assign=va, variant_update=vu)
        km2.set_stream(stream.cuda_stream)
        hp, hm = host_points.numpy(), host_means.numpy()   # (host_points exists: large shards skip this leg)
        out_means = torch.empty(k * dim, dtype=torch.float32).pin_memory()
        out_asg = torch.empty(count, dtype=torch.int32).pin_memory()
        km2.initialize(dim, k, count, 1, hp, hm)
        if world > 1:
            uid2 = torch.zeros(128, dtype=torch.uint8, device="cuda")
            if rank == 0:
                uid2.copy_(torch.frombuffer(bytearray(pkg.comm_unique_id()), dtype=torch.uint8))
            dist.broadcast(uid2, 0)
            km2.comm_init(bytes(uid2.cpu().numpy().tobytes()), world, rank)

        def e2e_step():
            # host -> device copy of points and means, preprocessing, one iteration, results back
            pkg.check(pkg.lib().bkm_initialize(km2._h, hp.ctypes.data, hm.ctypes.data))
            pkg.check(pkg.lib().bkm_run(km2._h, 1))
            pkg.check(pkg.lib().bkm_get_means(km2._h, out_means.data_ptr()))
            pkg.check(pkg.lib().bkm_get_assignment(km2._h, out_asg.data_ptr()))

        for _ in range(3):
            e2e_step()
        barrier()
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

    # ---------------- roofline of the dominant kernel (assignment) ----------------
    peaks = measured_peaks()
    flops_iter = 2.0 * count * k * dim            # algorithmic flops of one assignment launch on this rank
    bytes_iter = 4.0 * count * dim
    assign_ms = phases["assign"]
    roofline = None
    if assign_ms > 0:
        if counters["assign_variant"] == "tc" or flops_iter / (peaks["bf16_tflops"] * 0.5e12) > bytes_iter / (peaks["hbm_gbs"] * 1e9):
            tf32_peak = peaks["bf16_tflops"] * 0.5
            ach = flops_iter / (assign_ms * 1e-3) / 1e12
            traffic = C2_ASSIGN_TC_DRAM_BYTES if (args.workload == "c2" and not args.n and counters["assign_variant"] == "tc") else None
            roofline = {"bound": "tensor", "achieved": ach, "peak": tf32_peak, "unit": "TFLOP/s", "frac": ach / tf32_peak,
                        "traffic": traffic, "traffic_unit": "bytes per launch (ncu dram read+write, scaled from a quarter-size capture)",
                        "kernel": "assignment (%s)" % counters["assign_variant"],
                        "kernel_ms": assign_ms,
                        "peak_note": "TF32 dense taken as half the %s bf16 burst peak; 3xTF32 issues 3 tensor "
                                     "flops per algorithmic flop, so 1/3 is the ceiling of this fraction" % peaks["source"]}
        else:
            ach = bytes_iter / (assign_ms * 1e-3) / 1e9
            roofline = {"bound": "hbm", "achieved": ach, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                        "frac": ach / peaks["hbm_gbs"], "traffic": None,
                        "kernel": "assignment (%s)" % counters["assign_variant"], "kernel_ms": assign_ms,
                        "peak_note": "%s HBM copy bandwidth" % peaks["source"]}
    # the contractual whole-iteration roofline: slower of 2Nkd flops at peak and 4Nd bytes at HBM bandwidth
    t_roof = max(2.0 * count * k * dim / (peaks["bf16_tflops"] * 0.5e12), 4.0 * count * dim / (peaks["hbm_gbs"] * 1e9))
    iteration_roofline = {"roofline_ms": t_roof * 1e3, "frac": t_roof * 1e3 / ms_step,
                          "peaks": "tf32 = bf16/2 = %.1f TFLOP/s, hbm = %.1f GB/s (%s)" % (
                              peaks["bf16_tflops"] * 0.5, peaks["hbm_gbs"], peaks["source"])}

    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        sample_n = min(spec["n"], max(1 << 12, (1 << 26) // (k * max(1, dim // 32 + (dim % 32 > 0)))))
        cpu_baseline, _ = cpu_reference_leg(workloads, spec, args.seed, sample_n, 1, 0)

    if rank == 0:
        line = {"metric": "k-means iteration throughput", "value": value, "unit": "G dist-evals/s",
                "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step,
                "higher_is_better": True, "scaling": scaling,
                "vs_baseline": value / V100_PUBLISHED_GEVALS if args.workload == "c2" else None,
                "vs_baseline_note": "reference's best published number for this shape: 25.45 ms = 84.4 G dist-evals/s on V100",
                "dtype": "f32", "data": "synthetic", "config": config, "e2e": e2e,
                "gpu_launches": counters["launches_per_iter"] * args.steps,
                "roofline": roofline, "iteration_roofline": iteration_roofline, "cpu_baseline": cpu_baseline,
                "clocks": clocks, "phases_ms": phases, "variants": counters,
                "ns_per_input_float": ms_step * 1e6 / (n_total * dim)}
        print(json.dumps(line))
    km.cleanup()
    if dist is not None:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
