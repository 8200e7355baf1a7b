"""Per-op throughput of the B200 plugin through its C ABI: the size and op sweep of the hot path.

Every line is one op at one size, timed with CUDA events on the plugin's stream (median of the
iterations after warm-up), reported as algorithmic GB/s: 12 bytes per element for a binary op with
two full operands, 8 for a unary op or a binary op with a broadcast operand, 4 for a reduction or a
fill (the reference's accounting, benchmarks/bench.py:166-170). Inputs are larger than L2 from
64 MiB up; smaller sizes measure the cache and launch latency and say so.

Usage:
  python -m pytorches_b200.opbench --op add --elements 268435456 --iters 20
  python -m pytorches_b200.opbench --sweep            # 1 MiB .. 4 GiB, powers of 4, all ops
  python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 -m pytorches_b200.opbench --op add,sum ...
Under torch.distributed.run every rank runs the op on its own shard of --elements elements PER GPU
(dim-0 sharding, weak scaling); elementwise ops need no exchange, full-tensor reductions end with the
shard layer's combine; the line reports the aggregate over all GPUs with the slowest rank's time.
Ops: add mul div (contiguous), add_row (x[N/1024,1024] + b[1,1024]), add_col (x[R,1024] + s[R,1]),
exp relu neg, sum mean max argmax (full tensor), sum_rows max_rows (rows of 2048), sum_cols, axpy, fill,
add_t (transposed operand).
"""

from __future__ import annotations

import argparse
import ctypes
import json
import statistics
import sys

import torch

import pytorches_b200
from pytorches_b200.abi import op
from pytorches_b200.core import Device, Operand, Tensor, broadcast_strides, run_op, run_op_into

OPS = ["add", "mul", "div", "add_row", "add_col", "add_t", "exp", "relu", "neg", "axpy", "fill",
       "sum", "mean", "max", "argmax", "sum_rows", "max_rows", "sum_cols"]


def build_case(name: str, n: int, dev: Device, group=None):
    """Returns (callable issuing the op once, algorithmic bytes). ``group``: a ShardGroup when several
    ranks each hold a shard of n elements; full-tensor reductions then include the cross-GPU combine."""
    uni = lambda shape, seed: Tensor.randn_on(shape, seed, dev)
    if name in ("add", "mul", "div"):
        a, b = uni([n], 31), uni([n], 32).exp()  # second operand positive: a safe divisor
        code = {"add": op.ADD, "mul": op.MUL, "div": op.DIV}[name]
        return (lambda: a.raw_binary(b, code)), 12 * n
    if name == "add_row":
        a, b = uni([n // 1024, 1024], 31), uni([1, 1024], 32)
        return (lambda: a.raw_binary(b, op.ADD)), 8 * n + 4096
    if name == "add_col":
        a, s = uni([n // 1024, 1024], 31), uni([n // 1024, 1], 32)
        return (lambda: a.raw_binary(s, op.ADD)), 8 * n + 4 * (n // 1024)
    if name == "add_t":  # a [R, C] operand stored as [C, R], read through strides (1, R)
        r = 2048
        c = n // r
        a, b = uni([c, r], 31), uni([r, c], 32)
        ops = lambda: [Operand(a, [r, c], [1, r]), Operand.contiguous(b)]
        return (lambda: run_op(dev, op.ADD, [0], ops(), [r, c])), 12 * n
    if name in ("exp", "relu", "neg"):
        a = uni([n], 31)
        code = {"exp": op.EXP, "relu": op.RELU, "neg": op.NEG}[name]
        return (lambda: a.raw_unary(code)), 8 * n
    if name == "axpy":
        a, b = uni([n], 31), uni([n], 32)
        return (lambda: a.axpy_(-0.01, b)), 12 * n
    if name == "fill":
        out = uni([n], 31)
        return (lambda: run_op_into(dev, op.FILL, [0x3F800000], [], out.buffer, [n])), 4 * n
    if name in ("sum", "mean", "max", "argmax"):
        a = uni([n], 31 + (group.rank if group else 0))
        if group is not None and group.world > 1:
            calls = {"sum": lambda: group.sum(a), "mean": lambda: group.mean(a, n * group.world), "max": lambda: group.max(a),
                     "argmax": lambda: group.argmax(a, group.rank * n)}
            call = calls[name]

            def sharded():
                call()
                group.flush()  # the deferred combine belongs to this op's time

            return sharded, 4 * n
        return getattr(a, name), 4 * n
    if name in ("sum_rows", "max_rows"):
        a = uni([n // 2048, 2048], 31)
        return (lambda: a.sum_dim(1)) if name == "sum_rows" else (lambda: a.max_dim(1)), 4 * n + 4 * (n // 2048)
    if name == "sum_cols":
        a = uni([n // 4096, 4096], 31)
        return (lambda: a.sum_dim(0)), 4 * n + 4 * 4096
    raise SystemExit(f"unknown op {name}; choose from {OPS}")


def time_case(fn, stream, dev: Device, iters: int, warmup: int) -> float:
    for _ in range(warmup):
        fn()
    dev.synchronize()
    pairs = []
    for _ in range(iters):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(stream)
        fn()
        b.record(stream)
        pairs.append((a, b))
    dev.synchronize()
    torch.cuda.synchronize()
    return statistics.median(a.elapsed_time(b) for a, b in pairs)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--op", default="sum")
    ap.add_argument("--elements", type=int, default=1 << 28)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--device", type=int, default=0)
    ap.add_argument("--sweep", action="store_true")
    ap.add_argument("--peer", action="store_true",
                    help="sharded runs: exchange the per-GPU results inside the reduction kernels over peer memory instead of NCCL")
    ap.add_argument("--peak", type=float, default=6454.6, help="HBM GB/s the fraction is quoted against")
    args = ap.parse_args()

    import os

    world, rank = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0"))
    if world > 1:
        args.device = int(os.environ.get("LOCAL_RANK", "0"))
    plugin = pytorches_b200.load_plugin()
    if plugin.device_count() <= args.device:
        raise SystemExit("no CUDA device: the B200 plugin has no fallback")
    dev = Device(plugin, args.device)
    group = None
    if world > 1:
        import torch.distributed as dist

        from pytorches_b200.shard import ShardGroup, nccl_options

        torch.cuda.set_device(args.device)
        dist.init_process_group("nccl", device_id=torch.device("cuda", args.device), pg_options=nccl_options())
        group = ShardGroup(dev, rank, world)
        if args.peer and not group.enable_peer_exchange():
            raise SystemExit("in-kernel peer exchange could not be set up: " + plugin.last_error())
    get_stream = plugin.lib.pytorches_b200_stream
    get_stream.restype, get_stream.argtypes = ctypes.c_void_p, [ctypes.c_uint32]
    torch.cuda.set_device(args.device)
    stream = torch.cuda.ExternalStream(get_stream(args.device), device=torch.device("cuda", args.device))

    cases = [(name, args.elements) for name in (OPS if args.op == "all" else args.op.split(","))]
    if args.sweep:
        cases = [(name, (1 << 18) * 4 ** k) for name in OPS for k in range(7)]
    for name, n in cases:
        fn, nbytes = build_case(name, n, dev, group)
        if world > 1:
            dist.barrier()
        ms = time_case(fn, stream, dev, args.iters, args.warmup)
        if world > 1:  # the slowest rank's time, the bytes of all ranks
            t = torch.tensor([ms], dtype=torch.float64, device=f"cuda:{args.device}")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms, nbytes = float(t.item()), nbytes * world
        gbs = nbytes / (ms * 1e-3) / 1e9
        if rank == 0:
            print(json.dumps({"op": name, "gpus": world, "elements": n * world, "bytes": nbytes, "ms": round(ms, 5), "GB/s": round(gbs, 1),
                              "frac_of_peak": round(gbs / (args.peak * world), 4), "frac_of_8TBps": round(gbs / (8000.0 * world), 4),
                              "larger_than_l2": nbytes > 126e6 * world}))
            sys.stdout.flush()
        del fn
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
