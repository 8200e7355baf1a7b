"""Per-op throughput of the B200 plugin through its C ABI: the size and op sweep of the hot path.

Method (the reference's, benchmarks/bench.py:24-45): a run is FOUR enqueues of the op followed by a
synchronize; the figure is the median run after a warm-up, as algorithmic GB/s: 12 bytes per element
for a binary op with two full operands, 8 for a unary op or a binary op with a broadcast operand, 4
for a reduction or a fill (benchmarks/bench.py:166-170). Runs are timed with CUDA events on the
plugin's stream. The four enqueues of a run read four different copies of the operands when the
operands are smaller than 512 MiB, so that from 64 MiB up no enqueue finds its input in L2 (126 MB);
smaller sizes measure the cache and launch latency and the line says so. The enqueues are issued by
native code: one run goes through the Python mirror of the reference core once, is written down, and
is replayed (``pytorches_b200.replay``); ``--python`` keeps the Python mirror in the loop instead.

Values: uniform[0.5, 2) from the counter hash, seed 31 for the first operand, 32 for the second,
generated on the device by the appended RAND_UNIFORM op (the same bytes ``synth.uniform`` gives).

Usage:
  python -m pytorches_b200.opbench --op add --elements 268435456
  python -m pytorches_b200.opbench --sweep            # 1 MiB .. 8 GiB, all ops
  python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 -m pytorches_b200.opbench --op add,sum ...
Under torch.distributed.run the tensor of --elements elements is split along dim 0 over the ranks
(a fixed total size: strong scaling); elementwise ops need no exchange, full-tensor reductions end
with the cross-GPU combine inside their kernels; the line reports the whole job with the slowest
rank's time, against N x the per-GPU roofline.
Ops: add mul div (contiguous), add_row (x[N/1024,1024] + b[1,1024]), add_col (x[R,1024] + s[R,1]),
exp relu neg log tanh, sum mean max argmax (full tensor), sum_rows max_rows (rows of 2048), sum_cols
(4096 columns), axpy, fill, add_t (transposed operand).
"""

from __future__ import annotations

import argparse
import ctypes
import json
import os
import statistics
import sys
import time

import torch

import pytorches_b200
from pytorches_b200.abi import op
from pytorches_b200.core import Device, Operand, Tensor, run_op, run_op_into
from pytorches_b200.replay import Recorder

OPS = ["add", "mul", "div", "add_row", "add_col", "add_t", "exp", "relu", "neg", "log", "tanh", "axpy", "fill",
       "sum", "mean", "max", "argmax", "sum_rows", "max_rows", "sum_cols"]
ENQUEUES_PER_RUN = 4
ROTATE_BYTES = 512 << 20


def build_case(name: str, n: int, dev: Device, copies: int, group=None, n_total: int = 0, first: int = 0):
    """Returns (enqueue(j): issues the op once on copy j of its operands, algorithmic bytes of one
    enqueue on this rank, bytes of operands one copy holds). ``group``: a ShardGroup with the
    in-kernel exchange when the tensor is split over ranks; ``first`` = this rank's first element."""
    uni = lambda shape, seed, lo=0.5, hi=2.0: [Tensor.rand_uniform_on(shape, seed, lo, hi, dev, first) for _ in range(copies)]
    pick = lambda ts, j: ts[j % copies]
    if name in ("add", "mul", "div"):
        a, b = uni([n], 31), uni([n], 32)
        code = {"add": op.ADD, "mul": op.MUL, "div": op.DIV}[name]
        return (lambda j: pick(a, j).raw_binary(pick(b, j), code)), 12 * n, 8 * n
    if name == "add_row":
        a, b = uni([n // 1024, 1024], 31), Tensor.rand_uniform_on([1, 1024], 32, 0.5, 2.0, dev)
        return (lambda j: pick(a, j).raw_binary(b, op.ADD)), 8 * n + 4096, 4 * n
    if name == "add_col":
        a, s = uni([n // 1024, 1024], 31), uni([n // 1024, 1], 32)
        return (lambda j: pick(a, j).raw_binary(pick(s, j), op.ADD)), 8 * n + 4 * (n // 1024), 4 * n
    if name == "add_t":  # a [R, C] operand stored as [C, R], read through strides (1, R)
        r = 2048
        c = n // r
        a, b = uni([c, r], 31), uni([r, c], 32)
        ops = lambda j: [Operand(pick(a, j), [r, c], [1, r]), Operand.contiguous(pick(b, j))]
        return (lambda j: run_op(dev, op.ADD, [0], ops(j), [r, c])), 12 * n, 8 * n
    if name in ("exp", "relu", "neg", "log", "tanh"):
        a = uni([n], 31, -1.0, 1.0) if name in ("relu", "neg") else uni([n], 31)
        code = {"exp": op.EXP, "relu": op.RELU, "neg": op.NEG, "log": op.LOG, "tanh": op.TANH}[name]
        return (lambda j: pick(a, j).raw_unary(code)), 8 * n, 4 * n
    if name == "axpy":
        a, b = uni([n], 31), uni([n], 32)
        return (lambda j: pick(a, j).axpy_(-0.01, pick(b, j))), 12 * n, 8 * n
    if name == "fill":
        out = uni([n], 31)
        return (lambda j: run_op_into(dev, op.FILL, [0x3F800000], [], pick(out, j).buffer, [n])), 4 * n, 4 * n
    if name in ("sum", "mean", "max", "argmax"):
        a = uni([n], 31)
        if group is not None and group.world > 1:
            calls = {"sum": lambda j: group.sum(pick(a, j)), "mean": lambda j: group.mean(pick(a, j), n_total),
                     "max": lambda j: group.max(pick(a, j)), "argmax": lambda j: group.argmax(pick(a, j), first)}
            return calls[name], 4 * n, 4 * n
        return (lambda j: getattr(pick(a, j), name)()), 4 * n, 4 * n
    if name in ("sum_rows", "max_rows"):
        a = uni([n // 2048, 2048], 31)
        return ((lambda j: pick(a, j).sum_dim(1)) if name == "sum_rows" else (lambda j: pick(a, j).max_dim(1))), 4 * n + 4 * (n // 2048), 4 * n
    if name == "sum_cols":
        a = uni([n // 4096, 4096], 31)
        return (lambda j: pick(a, j).sum_dim(0)), 4 * n + 4 * 4096, 4 * n
    raise SystemExit(f"unknown op {name}; choose from {OPS}")


def copies_for(name: str, n: int, free_bytes: int) -> int:
    per_copy = {"add": 8, "mul": 8, "div": 8, "add_t": 8, "axpy": 8}.get(name, 4) * n
    want = max(1, min(ENQUEUES_PER_RUN, -(-ROTATE_BYTES // per_copy)))
    while want > 1 and want * per_copy > free_bytes // 3:
        want -= 1
    return want


def time_case(run, stream, dev: Device, iters: int, warmup_s: float) -> float:
    """Median device time of one run (four enqueues), each run bracketed by events and followed by a synchronize."""
    t0 = time.perf_counter()
    done = 0
    while done < 3 or time.perf_counter() - t0 < warmup_s:
        run()
        dev.synchronize()
        done += 1
    times = []
    for _ in range(iters):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(stream)
        run()
        b.record(stream)
        dev.synchronize()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b))
    return statistics.median(times)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--op", default="sum")
    ap.add_argument("--elements", type=int, default=1 << 28, help="elements of the whole tensor (split over the ranks when there are several)")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup-seconds", type=float, default=0.3)
    ap.add_argument("--device", type=int, default=0)
    ap.add_argument("--sweep", action="store_true", help="1 MiB .. 4 GiB in powers of 4, plus 8 GiB, every op")
    ap.add_argument("--python", action="store_true", help="issue the enqueues from the Python mirror of the core instead of replaying them natively")
    ap.add_argument("--peak", type=float, default=6454.6, help="HBM GB/s per GPU the fraction is quoted against")
    args = ap.parse_args()

    world, rank = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0"))
    if world > 1:
        args.device = int(os.environ.get("LOCAL_RANK", "0"))
    plugin = pytorches_b200.load_plugin()
    if plugin.device_count() <= args.device:
        raise SystemExit("no CUDA device: the B200 plugin has no fallback")
    recorder = Recorder(plugin)
    dev = Device(recorder, args.device)
    group = None
    torch.cuda.set_device(args.device)
    if world > 1:
        import torch.distributed as dist

        from pytorches_b200.shard import ShardGroup, nccl_options

        dist.init_process_group("nccl", device_id=torch.device("cuda", args.device), pg_options=nccl_options())
        group = ShardGroup(dev, rank, world)
        if not group.enable_peer_exchange():
            raise SystemExit("in-kernel peer exchange could not be set up: " + plugin.last_error())
    get_stream = plugin.lib.pytorches_b200_stream
    get_stream.restype, get_stream.argtypes = ctypes.c_void_p, [ctypes.c_uint32]
    stream = torch.cuda.ExternalStream(get_stream(args.device), device=torch.device("cuda", args.device))

    cases = [(name, args.elements) for name in (OPS if args.op == "all" else args.op.split(","))]
    if args.sweep:
        sizes = [(1 << 18) * 4 ** k for k in range(7)] + [1 << 31]
        cases = [(name, n) for name in OPS for n in sizes]
    try:
        for name, n_total in cases:
            n = n_total // world
            if name in ("add_row", "add_col", "sum_rows", "max_rows", "sum_cols", "add_t") and n % 4096:
                continue  # the 2-D shapes need whole rows on every rank
            free = plugin.device_info(args.device).free_memory
            copies = copies_for(name, n, free)
            need = {"add": 12, "mul": 12, "div": 12, "add_t": 12, "axpy": 8, "exp": 8, "relu": 8, "neg": 8, "log": 8, "tanh": 8,
                    "add_row": 8, "add_col": 8}.get(name, 4) * n
            if need + (copies - 1) * 4 * n > free * 0.9:
                if rank == 0:
                    print(json.dumps({"op": name, "gpus": world, "elements": n_total, "skipped": "does not fit in device memory"}))
                continue
            enqueue, nbytes, _ = build_case(name, n, dev, copies, group, n_total, rank * n)
            dev.synchronize()
            if args.python or (group is not None and not group.peer_exchange):
                def run():
                    for j in range(ENQUEUES_PER_RUN):
                        enqueue(j)
                driven = "Python mirror of the core"
            else:
                recorder.start()
                outs = [enqueue(j) for j in range(ENQUEUES_PER_RUN)]
                del outs
                rec = recorder.finish(args.device)
                dev.synchronize()

                def run(rec=rec):
                    if group is not None:
                        group.advance_peer_seq(rec.run(1, group.peer_seq))
                    else:
                        rec.run(1)
                driven = "recorded calls replayed natively"
            if world > 1:
                dist.barrier()
            ms = time_case(run, stream, dev, args.iters, args.warmup_seconds) / ENQUEUES_PER_RUN
            if world > 1:  # the slowest rank's time, the bytes of all ranks
                t = torch.tensor([ms], dtype=torch.float64, device=f"cuda:{args.device}")
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                ms, nbytes = float(t.item()), nbytes * world
            gbs = nbytes / (ms * 1e-3) / 1e9
            if rank == 0:
                print(json.dumps({"op": name, "gpus": world, "elements": n_total, "bytes": nbytes, "ms": round(ms, 5), "GB/s": round(gbs, 1),
                                  "frac_of_peak": round(gbs / (args.peak * world), 4), "frac_of_8TBps": round(gbs / (8000.0 * world), 4),
                                  "operand_copies_in_rotation": copies, "beyond_l2": copies * 4 * n >= 2 * 126_000_000 or 4 * n >= 2 * 126_000_000,
                                  "run": f"{ENQUEUES_PER_RUN} enqueues then a synchronize, median of {args.iters}", "driven_by": driven}))
                sys.stdout.flush()
            del enqueue, run
    finally:
        if world > 1:
            dist.destroy_process_group()


if __name__ == "__main__":
    main()
