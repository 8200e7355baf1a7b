"""Benchmark of the hot path: full-tensor f32 reductions through the plugin's C ABI.

Workload (the configuration the headline metric is quoted on): x = 2^28 f32 elements (1 GiB) per
GPU, uniform[-1, 1) from a counter hash with seed 7; one step = sum, mean, max and argmax (i64) of
x, each as the reference core would issue it (``Tensor::sum`` = reshape + SUM_AXIS, ``mean`` = that
plus a DIV by a scalar tensor). With N > 1 GPUs (one process per GPU) every rank holds its own
2^28-element shard of a 2^28*N-element tensor (weak scaling) and each op ends with the cross-GPU
combine of ``pytorches_b200.shard`` (all-gather of per-rank partials over NCCL, combined by plugin
ops). Algorithmic bytes: 4*n per op, so 4 GiB per step per GPU.

Prints ONE JSON line. ``value`` is device-resident throughput (CUDA events on the plugin's stream,
max over ranks); ``e2e`` is the same step fed from pinned host memory through ``copy_from_host`` with
the results read back; ``roofline`` is the SUM_AXIS launch (the dominant kernel) against the measured
HBM copy peak; ``cpu_baseline`` is the CPU oracle (a C++ restatement of the reference's CPU plugin,
which is Rust and cannot be built here) timed on this host's cores.

``--impl reference`` times that CPU implementation alone, on the same workload and metric.
"""

from __future__ import annotations

import argparse
import ctypes
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import numpy as np

N_ELEMS = 1 << 28
OPS = ("sum", "mean", "max", "argmax")
ORACLE_SO = os.path.join(ROOT, "oracle", "_build", "pytorches_plugin_cpuref.so")
METRIC = "f32 elementwise/reduce HBM GB/s"
# dram__bytes_read.sum + dram__bytes_write.sum of sum_rows_tma_kernel from the ncu capture summarised in
# profiles/sum_rows_tma_kernel_256mib.md (2^26 elements: 268.495 MB read, 5.07 MB written back from L2),
# read part scaled by 4 to this workload's 2^28 elements, write part kept.
NCU_TRAFFIC_PER_LAUNCH = int(268.495e6 * 4 + 5.07e6)


def uniform_pm1(n: int, seed: int, out: np.ndarray | None = None, first: int = 0) -> np.ndarray:
    """uniform[-1, 1) for counters first..first+n: u = (splitmix64(seed ^ i*GOLDEN) >> 40) / 2^24, value =
    2u - 1 (the counter hash of the ABI's RAND_NORMAL, crates/plugin-abi/src/lib.rs:101-107). Generated in
    slices to bound memory."""
    out = np.empty(n, dtype=np.float32) if out is None else out
    G = np.uint64(0x9E3779B97F4A7C15)
    step = 1 << 24
    with np.errstate(over="ignore"):
        for lo in range(0, n, step):
            i = np.arange(lo, min(lo + step, n), dtype=np.uint64) + np.uint64(first)
            x = np.uint64(seed) ^ (i * G)
            x = x + G
            x = (x ^ (x >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
            x = (x ^ (x >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
            x = x ^ (x >> np.uint64(31))
            u = (x >> np.uint64(40)).astype(np.float32) / np.float32(16777216.0)
            out[lo:lo + i.size] = np.float32(2.0) * u - np.float32(1.0)
    return out


def measured_peak_gbs() -> tuple[float, str]:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML while the timed region runs."""

    def __init__(self, index: int):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _run(self):
        nv = self.nv
        names = {
            getattr(nv, "nvmlClocksThrottleReasonHwSlowdown", 0x8): "hw_slowdown",
            getattr(nv, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
            getattr(nv, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
            getattr(nv, "nvmlClocksThrottleReasonSwPowerCap", 0x4): "sw_power_cap",
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.005)

    def __enter__(self):
        if self.nv:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread:
            self._thread.join()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons)}
        return {"sm_mhz": statistics.median(self.samples), "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(self.samples)}


def cpu_step(dev, x):
    return [x.sum(), x.mean(), x.max(), x.argmax()]


def run_cpu_baseline(max_seconds: float, min_steps: int = 2, fixed_steps: int | None = None, warmup: int = 1):
    """Times the CPU oracle on the full workload (all host threads). Returns (GB/s, cores, steps, seconds/step)."""
    from pytorches_b200.abi import Plugin
    from pytorches_b200.core import Device, Tensor

    oracle = Plugin(ORACLE_SO)
    threads = oracle.lib.cpuref_threads
    threads.restype = ctypes.c_uint
    dev = Device(oracle, 0)
    x = Tensor.from_numpy(uniform_pm1(N_ELEMS, 7), dev)
    for _ in range(max(warmup, 1)):
        cpu_step(dev, x)
    times = []
    t_begin = time.perf_counter()
    while True:
        t = time.perf_counter()
        cpu_step(dev, x)
        times.append(time.perf_counter() - t)
        if fixed_steps is not None:
            if len(times) >= fixed_steps:
                break
        elif len(times) >= min_steps and time.perf_counter() - t_begin >= max_seconds:
            break
    per_step = sum(times) / len(times)
    return len(OPS) * 4 * N_ELEMS / per_step / 1e9, int(threads()), len(times), per_step


def reference_arm(args):
    """The reference's CPU implementation of the path (the oracle port), alone."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    gbs, cores, steps, per_step = run_cpu_baseline(0.0, fixed_steps=args.steps, warmup=args.warmup)
    sample = f"full workload (sum, mean, max, argmax over 2^28 f32), {steps} steps on {cores} host threads"
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": round(gbs, 3), "unit": "GB/s", "n_gpus": args.gpus, "steps": steps,
        "warmup": args.warmup, "ms_per_step": round(per_step * 1e3, 3), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "config 2: full-tensor f32 sum/mean/max/argmax over 2^28 elements (1 GiB)", "elements": N_ELEMS,
                   "ops": list(OPS), "note": "C++ restatement of the reference's Rust CPU plugin (the reference cannot be built on this box)"},
        "cpu_baseline": {"value": round(gbs, 3), "unit": "GB/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": round(gbs, 3), "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--cpu-seconds", type=float, default=12.0, help="how long the cpu_baseline leg may run")
    ap.add_argument("--e2e-steps", type=int, default=5)
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        return reference_arm(args)

    # Libraries (NCCL's version banner, for one) print to stdout; the contract is ONE JSON line there.
    # Everything else goes to stderr: keep the real stdout aside for the final line.
    sys.stdout.flush()
    real_stdout = os.dup(1)
    os.dup2(2, 1)

    import torch
    import torch.distributed as dist

    import pytorches_b200
    from pytorches_b200.core import Device, Tensor
    from pytorches_b200.shard import ShardGroup, nccl_options

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE is {world}: launch one process per GPU (torch.distributed.run)")
    plugin = pytorches_b200.load_plugin()
    if plugin.device_count() <= local:
        raise SystemExit(f"the B200 plugin sees {plugin.device_count()} device(s); rank needs device {local} (there is no CPU fallback)")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local), pg_options=nccl_options())
    dev = Device(plugin, local)
    group = ShardGroup(dev, rank, world)
    exchange = "NCCL all-gather of the partials, combined by plugin ops"
    get_stream = plugin.lib.pytorches_b200_stream
    get_stream.restype, get_stream.argtypes = ctypes.c_void_p, [ctypes.c_uint32]
    stream = torch.cuda.ExternalStream(get_stream(local), device=torch.device("cuda", local))
    launches = plugin.lib.pytorches_b200_kernel_launches
    launches.restype = ctypes.c_uint64

    # This rank's shard: elements [rank*2^28, (rank+1)*2^28) of the global tensor, in pinned host memory.
    n_global = N_ELEMS * world
    host = torch.empty(N_ELEMS, dtype=torch.float32, pin_memory=True)
    host_np = host.numpy()
    uniform_pm1(N_ELEMS, 7, host_np, first=rank * N_ELEMS)
    x = Tensor.from_numpy(host_np, dev)
    first = rank * N_ELEMS

    def step(t):
        if world == 1:
            return [t.sum(), t.mean(), t.max(), t.argmax()]
        return [group.sum(t), group.mean(t, n_global), group.max(t), group.argmax(t, first)]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        dev.synchronize()

    # ---- correctness gate before any timing: x's reductions against numpy on the host copy ----
    res = [r.numpy() for r in step(x)]
    if world == 1:
        ref_sum = host_np.astype(np.float64).sum()
        tol = 1e-5 * 28 * np.abs(host_np).astype(np.float64).sum()
        assert abs(float(res[0]) - ref_sum) <= tol, (res[0], ref_sum)
        assert float(res[2]) == float(host_np.max()) and int(res[3]) == int(host_np.argmax()), "max/argmax mismatch"

    # ---- N > 1: move the exchange into the reduction kernels (peer stores over NVLink, one launch per
    # reduction, no collective library on the data path) if it sets up on every rank AND reproduces the
    # NCCL path's results bit for bit here; otherwise stay on NCCL. PYTORCHES_B200_PEER_EXCHANGE=0 keeps NCCL. ----
    if world > 1 and os.environ.get("PYTORCHES_B200_PEER_EXCHANGE", "1") != "0":
        ok = group.enable_peer_exchange()
        if ok:
            try:
                again = [r.numpy() for r in step(x)]
                ok = all(a.tobytes() == b.tobytes() for a, b in zip(again, res))
            except Exception as e:  # a bounded wait ran out, or the call failed: the device stays usable
                print(f"rank {rank}: in-kernel exchange failed its check: {e}", file=sys.stderr)
                ok = False
            flags = [None] * world
            dist.all_gather_object(flags, ok)
            ok = all(flags)
        if ok:
            exchange = "inside the reduction kernels: peer stores into every rank's window, ordered combine in the same launch"
        else:
            group.disable_peer_exchange()
            print(f"rank {rank}: staying on the NCCL exchange", file=sys.stderr)

    # ---- timed region: K steps, device-resident input ----
    def timed_region():
        """Warm-up, then K timed steps. Returns None if a step failed or the last step's results are not
        the gate's (possible only with the in-kernel exchange: a peer wait that ran out)."""
        try:
            for _ in range(args.warmup):
                step(x)
            # Everything slow or uneven between ranks (NVML start-up, allocations of events) happens BEFORE the
            # barrier: a rank that starts its first timed reduction late makes every other rank wait for it there.
            sampler = ClockSampler(local)
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
            op_ev = []  # per-op event pairs for the SUM_AXIS launch (first op of each step)
            l0 = launches()
            barrier()
            with sampler as clocks:
                ev[0].record(stream)
                t_host = time.perf_counter()
                for k in range(args.steps):
                    if world == 1:
                        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                        e0.record(stream)
                        s = x.sum()
                        e1.record(stream)
                        op_ev.append((e0, e1))
                        r = [s, x.mean(), x.max(), x.argmax()]
                    else:
                        r = step(x)
                group.flush()  # combines still deferred behind the last local pass
                ev[1].record(stream)
                host_ms = (time.perf_counter() - t_host) * 1e3 / args.steps  # time the host needs to ENQUEUE one step
                barrier()
            l1 = launches()
            same = all(a.numpy().tobytes() == b.tobytes() for a, b in zip(r, res))  # after the timed region: the steps computed the gate's values
            return (ev, op_ev, l0, l1, clocks, host_ms) if same else None
        except pytorches_b200.abi.PluginError as e:
            print(f"rank {rank}: timed region failed: {e}", file=sys.stderr)
            return None

    timed = timed_region()
    if world > 1:
        flags = [None] * world
        dist.all_gather_object(flags, timed is not None)
        if not all(flags) and group.peer_exchange:  # every rank goes back to NCCL together and measures again
            print(f"rank {rank}: in-kernel exchange failed during the timed region; measuring with NCCL", file=sys.stderr)
            group.disable_peer_exchange()
            exchange = "NCCL all-gather of the partials, combined by plugin ops (the in-kernel exchange failed in this run)"
            try:
                dev.synchronize()
            except pytorches_b200.abi.PluginError:
                pass  # the deferred report of the failed wait, if this rank had not seen it yet
            timed = timed_region()
            dist.all_gather_object(flags, timed is not None)
        if not all(flags):
            raise SystemExit("the timed steps failed or did not reproduce the gate's results")
    elif timed is None:
        raise SystemExit("the timed steps failed or did not reproduce the gate's results")
    ev, op_ev, l0, l1, clocks, host_ms = timed
    ms = ev[0].elapsed_time(ev[1])
    t_ms = torch.tensor([ms], dtype=torch.float64, device=f"cuda:{local}")
    rank_ms = [ms]
    if world > 1:
        all_ms = [torch.zeros_like(t_ms) for _ in range(world)]
        dist.all_gather(all_ms, t_ms)
        rank_ms = [float(t.item()) for t in all_ms]
        dist.all_reduce(t_ms, op=dist.ReduceOp.MAX)
    ms = float(t_ms.item())
    bytes_per_step = len(OPS) * 4 * N_ELEMS * world
    value = bytes_per_step * args.steps / (ms * 1e-3) / 1e9

    # ---- N > 1: the same four passes on every rank with NO exchange, all ranks at once. The gap between
    # the sharded step and the slowest rank's local passes is what the exchange and the combines cost. ----
    local_ms = None
    if world > 1:
        k_local = min(args.steps, 20)
        barrier()
        la, lb = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        la.record(stream)
        for _ in range(k_local):
            r = [x.sum(), x.mean(), x.max(), x.argmax()]
        lb.record(stream)
        barrier()
        mine = torch.tensor([la.elapsed_time(lb) / k_local], dtype=torch.float64, device=f"cuda:{local}")
        every = [torch.zeros_like(mine) for _ in range(world)]
        dist.all_gather(every, mine)
        local_ms = [round(float(t.item()), 4) for t in every]

    # ---- per-op device times (N = 1): every op alone, K launches each, for the breakdown ----
    per_op = {}
    if world == 1:
        for name, fn in (("sum", x.sum), ("mean", x.mean), ("max", x.max), ("argmax", x.argmax)):
            pairs = []
            for _ in range(min(args.steps, 50)):
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record(stream)
                fn()
                b.record(stream)
                pairs.append((a, b))
            dev.synchronize()
            torch.cuda.synchronize()
            per_op[name] = statistics.mean(a.elapsed_time(b) for a, b in pairs)

    # ---- end to end: the same step from pinned host memory through copy_from_host, results read back ----
    e2e = None
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.e2e_steps):
        xe = Tensor.from_numpy(host_np, dev)        # host -> device, 1 GiB, inside the timed region
        out = [r.numpy() for r in step(xe)]         # blocking device -> host reads of the four results
        del xe
    barrier()
    e2e_s = (time.perf_counter() - t0) / args.e2e_steps
    t_e = torch.tensor([e2e_s], dtype=torch.float64, device=f"cuda:{local}")
    if world > 1:
        dist.all_reduce(t_e, op=dist.ReduceOp.MAX)
    e2e_s = float(t_e.item())
    e2e = {"value": round(bytes_per_step / e2e_s / 1e9, 3), "unit": "GB/s", "h2d_bytes_per_step": 4 * N_ELEMS * world,
           "d2h_bytes_per_step": (4 + 4 + 4 + 8) * world, "ms_per_step": round(e2e_s * 1e3, 3), "steps": args.e2e_steps}

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peak, peak_kind = measured_peak_gbs()
    roofline = None
    if op_ev:
        sum_ms = statistics.mean(a.elapsed_time(b) for a, b in op_ev)
        achieved = 4 * N_ELEMS / (sum_ms * 1e-3) / 1e9
        roofline = {"bound": "hbm", "kernel": "sum_rows_tma_kernel<fused>: one SUM_AXIS over 2^28 f32 (streaming pass with the ordered combine in the same launch)", "achieved": round(achieved, 1),
                    "peak": peak, "peak_kind": peak_kind, "unit": "GB/s", "frac": round(achieved / peak, 4), "frac_of_8TBps": round(achieved / 8000.0, 4),
                    "algorithmic_bytes_per_launch": 4 * N_ELEMS, "ms_per_launch": round(sum_ms, 5), "traffic": NCU_TRAFFIC_PER_LAUNCH}
    cpu = None
    if world == 1:
        gbs, cores, steps, per_step = run_cpu_baseline(args.cpu_seconds)
        cpu = {"value": round(gbs, 3), "unit": "GB/s", "cores": cores, "kind": "port",
               "sample": f"full workload, {steps} steps of {per_step * 1e3:.1f} ms on {cores} host threads (C++ restatement of the reference CPU plugin)"}
    line = {
        "metric": METRIC, "value": round(value, 1), "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms / args.steps, 5), "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": "config 2: full-tensor f32 sum/mean/max/argmax over 2^28 elements (1 GiB) per GPU", "elements_per_gpu": N_ELEMS,
                   "ops": list(OPS), "sharding": f"dim 0 over {world} GPU(s); exchange: {exchange}" if world > 1 else "none",
                   "l2": "input (1 GiB) is larger than L2 (126 MB); no flush needed", "frac_of_measured_peak": round(value / (peak * world), 4),
                   "frac_of_8TBps": round(value / (8000.0 * world), 4)},
        "clocks": clocks.summary(), "e2e": e2e, "gpu_launches": int(l1 - l0), "host_enqueue_ms_per_step": round(host_ms, 4), "rank_ms_per_step": [round(v / args.steps, 4) for v in rank_ms],
        "rank_local_ms_per_step_no_exchange": local_ms, "roofline": roofline, "cpu_baseline": cpu,
        "ops_ms": {k: round(v, 5) for k, v in per_op.items()}, "results": {"sum": float(res[0]), "mean": float(res[1]), "max": float(res[2]), "argmax": int(res[3])},
    }
    sys.stdout.flush()
    os.write(real_stdout, (json.dumps(line) + "\n").encode())
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
