"""Benchmark of the hot path: full-tensor f32 reductions through the plugin's C ABI.

Workload (the configuration the headline metric is quoted on): ONE tensor x of 2^28 f32 elements
(1 GiB), uniform[-1, 1) from the ABI's counter hash with seed 7; one step = sum, mean, max and argmax
(i64) of x, each as the reference core would issue it (``Tensor::sum`` = reshape + SUM_AXIS, ``mean`` =
that plus a DIV by a scalar tensor). With N > 1 GPUs (one process per GPU) the SAME tensor is split along
dim 0: rank r holds elements [r * 2^28/N, (r+1) * 2^28/N) (strong scaling), reduces its shard, and each
op ends with the cross-GPU combine of ``pytorches_b200.shard``, so every N computes the reductions of the
same 2^28 values. Algorithmic bytes: 4*n per op, 4 GiB per step for the whole job.

A shard of 2^28/N elements approaches the size of L2 (126 MB) at N = 8, so every rank keeps K copies
of its shard (K * shard >= 512 MiB) and consecutive ops read consecutive copies: an op never finds its
input in L2.

The timed region is driven by native code: one step is run once through the Python mirror of the
reference core, its plugin calls (alloc, execute, free, sharded reductions) are written down, and the
list is replayed through ``pytorches_b200_replay``, as a native host like the reference's core would
issue it. The Python mirror needs 10-25 us per op, as long as an op runs for on a 128 MiB shard.

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
import math
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import numpy as np

from pytorches_b200.synth import uniform_pm1

N_ELEMS = 1 << 28
OPS = ("sum", "mean", "max", "argmax")
ORACLE_SO = os.path.join(ROOT, "oracle", "_build", "pytorches_plugin_cpuref.so")
METRIC = "f32 elementwise/reduce HBM GB/s"
ROTATE_BYTES = 512 << 20  # an op's input was last touched at least this many bytes of traffic ago
# dram__bytes_read.sum + dram__bytes_write.sum of one fused SUM_AXIS launch, from an ncu capture of a
# 2^26-element launch (268.53 MB read, 4.05 MB written back from L2): the read part grows with the
# element count and is scaled to this workload's launch, the write part is kept.
NCU_READ_BYTES_PER_ELEMENT = 268.531712e6 / (1 << 26)
NCU_WRITE_BYTES_PER_LAUNCH = 4.047104e6


def workload_config(world: int) -> dict:
    """The ``config`` object, the same in both arms (the reference arm runs on this arm's config)."""
    return {
        "workload": "config 2: full-tensor f32 sum/mean/max/argmax over ONE tensor of 2^28 elements (1 GiB), uniform[-1,1) seed 7",
        "elements": N_ELEMS, "ops": list(OPS),
        "sharding": "none" if world == 1 else f"dim 0 over {world} GPUs, 2^28/{world} elements per GPU, partials combined across GPUs",
        "l2": "device arm: consecutive ops read consecutive copies of the (shard of the) tensor, copies x size >= 512 MiB, so no op finds "
              "its input in the 126 MB L2; at 1 and 2 GPUs the input itself is larger than L2",
    }


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
        "warmup": args.warmup, "ms_per_step": round(per_step * 1e3, 3), "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": workload_config(args.gpus),
        "note": "C++ restatement of the reference's Rust CPU plugin (the reference cannot be built on this box); host cores only, whatever --gpus says",
        "cpu_baseline": {"value": round(gbs, 3), "unit": "GB/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": round(gbs, 3), "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def host_reference(shard: np.ndarray, first: int) -> dict:
    """This rank's share of an independent check, from the host copy of its shard: f64 sum and sum of
    magnitudes, the maximum and the first global position where it occurs."""
    return {"sum": float(shard.sum(dtype=np.float64)), "abs": float(np.abs(shard).sum(dtype=np.float64)), "max": float(shard.max()),
            "argmax": first + int(shard.argmax())}


def check_against_host(res, parts: list[dict]) -> None:
    """Device results of the WHOLE tensor against the per-rank host values: sum and mean within the
    stated tolerance (relative 1e-5 * log2 n of the sum of magnitudes), max and argmax exactly (the lowest
    global position among equal maxima)."""
    total, mag = sum(p["sum"] for p in parts), sum(p["abs"] for p in parts)
    tol = 1e-5 * math.log2(N_ELEMS) * mag
    best = max(p["max"] for p in parts)
    where = min(p["argmax"] for p in parts if p["max"] == best)
    assert abs(float(res[0]) - total) <= tol, ("sum", float(res[0]), total, tol)
    assert abs(float(res[1]) - total / N_ELEMS) <= tol / N_ELEMS, ("mean", float(res[1]), total / N_ELEMS)
    assert float(res[2]) == best, ("max", float(res[2]), best)
    assert int(res[3]) == where, ("argmax", int(res[3]), where)


def oracle_shard_sums(shard: np.ndarray):
    """From the CPU oracle (None if it has not been built; checker only): its SUM_AXIS of this rank's
    shard, and its sums of the shard's 65536-element blocks (the units the reference chains in block
    order, plugins/cpu/src/reduce.rs:110-131)."""
    if not os.path.exists(ORACLE_SO):
        return None
    from pytorches_b200.abi import Plugin
    from pytorches_b200.core import Device, Tensor

    dev = Device(Plugin(ORACLE_SO), 0)
    t = Tensor.from_numpy(shard, dev)
    whole = float(t.sum().numpy().reshape(()))
    blocks = t.raw_reshape([shard.size // 65536, 65536]).raw_sum_axis(1).numpy() if shard.size % 65536 == 0 else None
    return whole, blocks


def chain_f32(values) -> np.float32:
    """((0 + v0) + v1) + ... in f32, the reference's combine of block sums."""
    acc = np.float32(0.0)
    for v in values:
        acc = np.float32(acc + np.float32(v))
    return acc


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--cpu-seconds", type=float, default=12.0, help="how long the cpu_baseline leg may run")
    ap.add_argument("--e2e-steps", type=int, default=5)
    ap.add_argument("--min-seconds", type=float, default=0.5, help="the timed region repeats the K steps until it lasts at least this long")
    ap.add_argument("--warmup-seconds", type=float, default=1.0, help="warm-up continues until this much time has passed")
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
    from pytorches_b200.replay import Recorder
    from pytorches_b200.shard import ShardGroup, nccl_options

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE is {world}: launch one process per GPU (torch.distributed.run)")
    if N_ELEMS % world:
        raise SystemExit(f"2^28 elements do not split evenly over {world} GPUs")
    plugin = pytorches_b200.load_plugin()
    if plugin.device_count() <= local:
        raise SystemExit(f"the B200 plugin sees {plugin.device_count()} device(s); rank needs device {local} (there is no CPU fallback)")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local), pg_options=nccl_options())
    try:
        line = run(args, plugin, rank, world, local, torch, dist, Device, Tensor, Recorder, ShardGroup)
    finally:
        if world > 1:
            dist.destroy_process_group()
    if line is not None:
        sys.stdout.flush()
        os.write(real_stdout, (json.dumps(line) + "\n").encode())


def run(args, plugin, rank, world, local, torch, dist, Device, Tensor, Recorder, ShardGroup):
    import pytorches_b200

    recorder = Recorder(plugin)
    dev = Device(recorder, local)
    group = ShardGroup(dev, rank, world)
    exchange = "NCCL all-gather of the partials, combined by plugin ops"
    get_stream = plugin.lib.pytorches_b200_stream
    get_stream.restype, get_stream.argtypes = ctypes.c_void_p, [ctypes.c_uint32]
    stream = torch.cuda.ExternalStream(get_stream(local), device=torch.device("cuda", local))
    launches = plugin.lib.pytorches_b200_kernel_launches
    launches.restype = ctypes.c_uint64

    # This rank's shard of THE tensor: counters [first, first + n_local) of the seed-7 stream, in pinned host memory.
    n_local = N_ELEMS // world
    first = rank * n_local
    host = torch.empty(n_local, dtype=torch.float32, pin_memory=True)
    host_np = host.numpy()
    uniform_pm1(n_local, 7, host_np, first=first)
    copies = max(1, -(-ROTATE_BYTES // (4 * n_local)))
    xs = [Tensor.from_numpy(host_np, dev) for _ in range(copies)]

    def step(pick):
        """One step; ``pick(j)`` is the tensor op j reads (the same values in every copy)."""
        if world == 1:
            return [pick(0).sum(), pick(1).mean(), pick(2).max(), pick(3).argmax()]
        # With the in-kernel exchange on, sum and mean are taken in UNSPLIT order (the shards are whole
        # 65536-element blocks): the bits of the one-GPU result at every N.
        return [group.sum(pick(0), first, N_ELEMS), group.mean(pick(1), N_ELEMS, first), group.max(pick(2)), group.argmax(pick(3), first)]

    rotating = lambda j: xs[j % copies]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        dev.synchronize()

    def gather(obj):
        if world == 1:
            return [obj]
        every = [None] * world
        dist.all_gather_object(every, obj)
        return every

    # ---- correctness gate before any timing, at every N: the device's results for the whole tensor against
    # (a) numpy in f64 on the host shards and (b) the CPU oracle's per-shard sums combined in rank order ----
    parts = gather(host_reference(host_np, first))
    res = [r.numpy() for r in step(rotating)]  # N > 1: through NCCL, per-rank results combined in rank order
    check_against_host(res, parts)
    checks = {"vs_host_f64": True}
    mine = oracle_shard_sums(host_np)
    every = gather(mine)
    want_unsplit = None
    if all(m is not None for m in every):
        if world == 1:
            want = np.float32(every[0][0])
        else:  # SUM_AXIS over the [world] tensor of per-rank sums: added one by one to 0.0, then 0.0 + that
            want = np.float32(np.float32(0.0) + chain_f32(m[0] for m in every))
        assert np.float32(res[0]).tobytes() == want.tobytes(), ("sum differs from the oracle's rank-ordered combine", float(res[0]), float(want))
        assert np.float32(res[1]).tobytes() == np.float32(want / np.float32(N_ELEMS)).tobytes(), "mean differs from the oracle's"
        checks["sum_mean_bit_equal_to_oracle_rank_ordered"] = True
        if all(m[1] is not None for m in every):  # the oracle's sum over the UNSPLIT tensor: all block sums chained in block order
            want_unsplit = chain_f32(np.concatenate([m[1] for m in every]))
            if world == 1:
                assert want_unsplit.tobytes() == want.tobytes(), "the chain of the oracle's block sums is not the oracle's sum"

    # ---- N > 1: move the exchange into the reduction kernels (peer stores over NVLink, one launch per
    # reduction, no collective library on the data path) if it sets up on every rank AND passes its checks
    # here: max and argmax bit-equal to the NCCL path's, sum and mean (now in unsplit order) bit-equal to
    # the oracle's over the unsplit tensor and within tolerance of numpy; otherwise stay on NCCL.
    # PYTORCHES_B200_PEER_EXCHANGE=0 keeps NCCL. ----
    if world > 1 and os.environ.get("PYTORCHES_B200_PEER_EXCHANGE", "1") != "0":
        ok = group.enable_peer_exchange()
        again = None
        if ok:
            try:
                again = [r.numpy() for r in step(rotating)]
                check_against_host(again, parts)
                ok = again[2].tobytes() == res[2].tobytes() and again[3].tobytes() == res[3].tobytes()
                if ok and group.unsplit_order(N_ELEMS) and want_unsplit is not None:
                    ok = (np.float32(again[0]).tobytes() == want_unsplit.tobytes()
                          and np.float32(again[1]).tobytes() == np.float32(want_unsplit / np.float32(N_ELEMS)).tobytes())
                elif ok:
                    ok = again[0].tobytes() == res[0].tobytes() and again[1].tobytes() == res[1].tobytes()
            except Exception as e:  # a bounded wait ran out, a check failed, or the call failed: the device stays usable
                print(f"rank {rank}: in-kernel exchange failed its check: {e!r}", file=sys.stderr)
                ok = False
            ok = all(gather(ok))
        if ok:
            exchange = "inside the reduction kernels: peer stores into every rank's window, ordered combine in the same launch"
            checks["max_argmax_bit_equal_to_nccl_path"] = True
            if group.unsplit_order(N_ELEMS):
                exchange += "; sum and mean in unsplit order (every rank chains all 4096 block sums)"
                if want_unsplit is not None:
                    checks["sum_mean_bit_equal_to_oracle_unsplit"] = True
            res = again  # what the timed steps must reproduce
        else:
            group.disable_peer_exchange()
            print(f"rank {rank}: staying on the NCCL exchange", file=sys.stderr)
    elif world == 1 and want_unsplit is not None:
        checks["sum_mean_bit_equal_to_oracle_unsplit"] = True

    def record_step():
        """Runs one step for real through the recorder; returns (its call list, its results)."""
        group.flush()
        dev.synchronize()
        recorder.start()
        out = step(rotating)
        group.flush()
        got = [r.numpy() for r in out]
        del out
        return recorder.finish(local, keep=xs), got

    # ---- timed region: K steps (repeated until the region lasts long enough), device-resident input ----
    def timed_region():
        """Warm-up, then the timed passes. Returns None if a step failed or the steps' results are not the
        gate's (possible only with the in-kernel exchange: a peer wait that ran out)."""
        try:
            native = group.peer_exchange or world == 1  # the NCCL path's collectives are issued by torch: Python drives it
            rec, got = record_step() if native else (None, [r.numpy() for r in step(rotating)])
            if not all(a.tobytes() == b.tobytes() for a, b in zip(got, res)):
                return None

            def passes(k):
                if native:
                    group.advance_peer_seq(rec.run(k, group.peer_seq))
                else:
                    for _ in range(k):
                        step(rotating)
                    group.flush()

            passes(args.warmup)
            # Warm-up by time as well as by count; the same run tells how long one pass takes, which
            # sizes the timed region. Every rank must come to the same counts: rank 0's are used.
            barrier()
            t0 = time.perf_counter()
            probe = 0
            while True:
                passes(args.steps)
                dev.synchronize()
                probe += args.steps
                if all(gather(time.perf_counter() - t0 >= args.warmup_seconds)):
                    break
            per_pass = (time.perf_counter() - t0) / probe
            inner = gather(max(1, math.ceil(args.min_seconds / (per_pass * args.steps))))[0]
            groups = 20 if args.steps * inner >= 20 else 1
            total = args.steps * inner
            sizes = [total // groups + (1 if g < total % groups else 0) for g in range(groups)]
            # Everything slow or uneven between ranks (NVML start-up, allocations of events) happens BEFORE the
            # barrier: a rank that starts its first timed reduction late makes every other rank wait for it there.
            sampler = ClockSampler(local)
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(groups + 1)]
            l0 = launches()
            barrier()
            with sampler as clocks:
                ev[0].record(stream)
                t_host = time.perf_counter()
                for g, k in enumerate(sizes):  # an event between groups of passes: the median group is reported beside the total
                    passes(k)
                    ev[g + 1].record(stream)
                host_ms = (time.perf_counter() - t_host) * 1e3 / total  # time the host needs to ENQUEUE one step
                barrier()
            l1 = launches()
            trace = None
            if world > 1 and group.peer_exchange and os.environ.get("PYTORCHES_B200_PEER_TRACE") == "1":  # where the sharded reductions' time went, by the device's clock
                rec_t, last = group.peer_trace().astype(np.int64), group.peer_seq
                trace = {}
                rec_of = lambda q: rec_t[(q % 0xfffffffe + 1) % 64]
                for j, name in enumerate(OPS):  # reduction number q is op q % 4 of a step; its record is (q % 0xfffffffe + 1) % 64
                    qs = [q for q in range(max(last - 60, 1), last) if q % len(OPS) == j and rec_of(q)[1:4].min() > 0 and rec_of(q - 1)[3] > 0]
                    if not qs:
                        continue
                    med = lambda f: round(statistics.median(f(rec_of(q)) / 1e3 for q in qs), 2)
                    trace[name] = {"wait_for_slowest_peer_us": med(lambda r: r[2] - r[1]), "after_last_arrival_us": med(lambda r: r[3] - r[2]),
                                   "result_after_previous_result_us": round(statistics.median((rec_of(q)[3] - rec_of(q - 1)[3]) / 1e3 for q in qs), 2)}
                    if all(rec_of(q)[13] > 0 for q in qs):  # a sum in unsplit order: bulk copies of the block sums its combiner needed
                        trace[name]["combiner_copies"] = int(statistics.median(int(rec_of(q)[13]) for q in qs))
            # after the timed region: one more step, read back, must still be the gate's values
            same = all(a.numpy().tobytes() == b.tobytes() for a, b in zip(step(rotating), res))
            if not same:
                return None
            ms_total = ev[0].elapsed_time(ev[-1])
            per_group = [ev[g].elapsed_time(ev[g + 1]) / sizes[g] for g in range(groups)]
            return {"ms": ms_total, "passes": total, "inner": inner, "launches": int(l1 - l0), "clocks": clocks, "host_ms": host_ms,
                    "median_ms": statistics.median(per_group), "calls_per_pass": rec.executes if native else None, "trace": trace,
                    "driver": "recorded call list replayed by pytorches_b200_replay" if native else "Python mirror of the core"}
        except pytorches_b200.abi.PluginError as e:
            print(f"rank {rank}: timed region failed: {e}", file=sys.stderr)
            return None

    timed = timed_region()
    if world > 1:
        flags = gather(timed is not None)
        if not all(flags) and group.peer_exchange:  # every rank goes back to NCCL together and measures again
            print(f"rank {rank}: in-kernel exchange failed during the timed region; measuring with NCCL", file=sys.stderr)
            group.disable_peer_exchange()
            checks.pop("max_argmax_bit_equal_to_nccl_path", None)
            checks.pop("sum_mean_bit_equal_to_oracle_unsplit", None)
            exchange = "NCCL all-gather of the partials, combined by plugin ops (the in-kernel exchange failed in this run)"
            try:
                dev.synchronize()
            except pytorches_b200.abi.PluginError:
                pass  # the deferred report of the failed wait, if this rank had not seen it yet
            res = [r.numpy() for r in step(rotating)]  # the NCCL path's values are the ones to reproduce now
            timed = timed_region()
            flags = gather(timed is not None)
        if not all(flags):
            raise SystemExit("the timed steps failed or did not reproduce the gate's results")
    elif timed is None:
        raise SystemExit("the timed steps failed or did not reproduce the gate's results")
    ms = timed["ms"]
    traces = gather(timed["trace"]) if world > 1 else None
    t_ms = torch.tensor([ms], dtype=torch.float64, device=f"cuda:{local}")
    rank_ms = [ms]
    if world > 1:
        all_ms = [torch.zeros_like(t_ms) for _ in range(world)]
        dist.all_gather(all_ms, t_ms)
        rank_ms = [float(t.item()) for t in all_ms]
        dist.all_reduce(t_ms, op=dist.ReduceOp.MAX)
    ms = float(t_ms.item())
    bytes_per_step = len(OPS) * 4 * N_ELEMS  # the whole job: all ranks' shards together are the one tensor
    value = bytes_per_step * timed["passes"] / (ms * 1e-3) / 1e9

    # ---- N > 1: the same four passes on every rank with NO exchange, all ranks at once. The gap between
    # the sharded step and the slowest rank's local passes is what the exchange and the combines cost. ----
    local_ms = None
    if world > 1:
        recorder.start()
        out = [rotating(0).sum(), rotating(1).mean(), rotating(2).max(), rotating(3).argmax()]
        del out
        rec_local = recorder.finish(local, keep=xs)
        k_local = max(args.steps, 20)
        rec_local.run(args.warmup)
        barrier()
        la, lb = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        la.record(stream)
        rec_local.run(k_local)
        lb.record(stream)
        barrier()
        local_ms = [round(v, 4) for v in gather(la.elapsed_time(lb) / k_local)]

    # ---- the dominant kernel alone, and every op alone (N = 1): K launches each with an event pair around
    # every launch, for the roofline and the breakdown ----
    per_op, sum_ms = {}, None
    if world == 1:
        x = xs[0]
        for name, fn in (("sum", x.sum), ("mean", x.mean), ("max", x.max), ("argmax", x.argmax)):
            pairs = []
            for _ in range(min(max(args.steps, 20), 50)):
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record(stream)
                fn()
                b.record(stream)
                pairs.append((a, b))
            dev.synchronize()
            torch.cuda.synchronize()
            per_op[name] = statistics.mean(a.elapsed_time(b) for a, b in pairs)
        sum_ms = per_op["sum"]

    # ---- end to end: the same step from pinned host memory through copy_from_host, results read back ----
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.e2e_steps):
        xe = Tensor.from_numpy(host_np, dev)                 # host -> device, this rank's shard, inside the timed region
        out = [r.numpy() for r in step(lambda j: xe)]        # blocking device -> host reads of the four results
        del xe
    barrier()
    e2e_s = max(gather((time.perf_counter() - t0) / args.e2e_steps))
    assert all(a.tobytes() == b.tobytes() for a, b in zip(out, res)), "the end-to-end step's results differ from the gate's"
    e2e = {"value": round(bytes_per_step / e2e_s / 1e9, 3), "unit": "GB/s", "h2d_bytes_per_step": 4 * N_ELEMS,
           "d2h_bytes_per_step": (4 + 4 + 4 + 8) * world, "ms_per_step": round(e2e_s * 1e3, 3), "steps": args.e2e_steps}

    if rank != 0:
        return None

    peak, peak_kind = measured_peak_gbs()
    roofline = None
    if sum_ms:
        achieved = 4 * N_ELEMS / (sum_ms * 1e-3) / 1e9
        roofline = {"bound": "hbm", "kernel": "sum_rows_tma_kernel<fused>: one SUM_AXIS over 2^28 f32 (streaming pass with the ordered combine in the same launch)",
                    "achieved": round(achieved, 1), "peak": peak, "peak_kind": peak_kind, "unit": "GB/s", "frac": round(achieved / peak, 4),
                    "frac_of_8TBps": round(achieved / 8000.0, 4), "algorithmic_bytes_per_launch": 4 * N_ELEMS, "ms_per_launch": round(sum_ms, 5),
                    "timing": "mean over launches issued one by one with a CUDA event pair around each, after the timed region",
                    "traffic": int(NCU_READ_BYTES_PER_ELEMENT * N_ELEMS + NCU_WRITE_BYTES_PER_LAUNCH)}
    cpu = None
    if world == 1:
        gbs, cores, steps, per_step = run_cpu_baseline(args.cpu_seconds)
        cpu = {"value": round(gbs, 3), "unit": "GB/s", "cores": cores, "kind": "port",
               "sample": f"full workload, {steps} steps of {per_step * 1e3:.1f} ms on {cores} host threads (C++ restatement of the reference CPU plugin)"}
    passes = timed["passes"]
    return {
        "metric": METRIC, "value": round(value, 1), "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms / passes, 5), "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "config": workload_config(world),
        "method": {"inner_repeats": timed["inner"], "timed_steps": passes, "timed_region_ms": round(ms, 3),
                   "ms_per_step_median_of_groups": round(timed["median_ms"], 5), "copies_in_rotation": copies,
                   "bytes_in_rotation": copies * 4 * n_local, "driven_by": timed["driver"], "calls_per_step": timed["calls_per_pass"],
                   "exchange": exchange if world > 1 else "none", "warmup_seconds": args.warmup_seconds},
        "frac_of_measured_peak": round(value / (peak * world), 4), "frac_of_8TBps": round(value / (8000.0 * world), 4),
        "clocks": timed["clocks"].summary(), "e2e": e2e, "gpu_launches": timed["launches"], "host_enqueue_ms_per_step": round(timed["host_ms"], 5),
        "rank_ms_per_step": [round(v / passes, 5) for v in rank_ms], "rank_local_ms_per_step_no_exchange": local_ms,
        "exchange_trace_per_rank": traces,
        "roofline": roofline, "cpu_baseline": cpu, "ops_ms": {k: round(v, 5) for k, v in per_op.items()},
        "results": {"sum": float(res[0]), "mean": float(res[1]), "max": float(res[2]), "argmax": int(res[3])},
        "results_check": checks,
    }


if __name__ == "__main__":
    main()
