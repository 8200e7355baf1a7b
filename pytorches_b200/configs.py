"""The benchmark configurations of the hot path, run end to end through the plugin's C ABI.

Each configuration is issued the way the reference core would issue it (one ``execute`` per op, a fresh
output buffer per op, backward as plain ops), timed with CUDA events on the plugin's stream, and
reported as algorithmic GB/s. Algorithmic bytes are counted per ``execute`` from its descriptors: every
operand once at its STORED size (a broadcast operand counts the elements it really holds), the output
once (the reference's accounting: add = 3*4*n, sum = 4*n, benchmarks/bench.py:166-170).

  config 1  out = relu(A + b) * s; r = sum(out, dim=1); backward of sum(out): dA, db, ds   (A 4096x4096)
  config 3  elementwise part of an MLP step, widths [8192]*13, batch 32: 11 x ReLU fwd/bwd, mse_loss,
            SGD update p -= 0.01*g over 805M parameters (AXPY per tensor)
  config 4  softmax from primitives on X[64,2048,2048] with broadcast addends; also with X a transposed view
(config 2 is bench.py; config 5 is ``python -m pytorches_b200.opbench --sweep``.)

Each step is issued the way a native host would: it runs once through the Python mirror of the core, its
plugin calls are written down and then replayed by ``pytorches_b200_replay`` (``--python`` adds the
Python-driven figure for comparison). Config 3 shards by whole layers when launched under
``torch.distributed.run`` (12 layers over 8 GPUs is uneven: the ideal speed-up is 6.0, at 4 GPUs 4.0, at 2 2.0).

Usage:  python -m pytorches_b200.configs [--config 1,3,4,4t] [--iters 10] [--python] [--fused]
"""

from __future__ import annotations

import argparse
import ctypes
import json
import math
import os
import statistics
import sys
import time

import numpy as np

import pytorches_b200
from pytorches_b200 import synth
from pytorches_b200.abi import Plugin, op
from pytorches_b200.core import SGD, Device, Operand, Tensor, broadcast_strides, mse_loss, run_op


def config1(dev: Device):
    A = Tensor.randn_on([4096, 4096], 1, dev).requires_grad_()
    b = Tensor.randn_on([1, 4096], 2, dev).requires_grad_()
    s = Tensor.randn_on([4096, 1], 3, dev).requires_grad_()

    def step():
        for t in (A, b, s):
            t.grad = None
        out = A.add_relu(b) * s  # ADD then RELU (and STEP then MUL in backward) unless the device uses the fused ops
        r = out.sum_dim(1)
        out.sum().backward()
        return r, A.grad, b.grad, s.grad

    return step


def config3(dev: Device, layers: int = 12, width: int = 8192, batch: int = 32):
    params, grads = [], []
    for l in range(layers):
        for shape, k in (([width, width], 0), ([width], 1)):
            p = Tensor.randn_on(shape, 11 + 100 * l + k, dev).raw_binary(Tensor.scalar_on(0.02, dev), op.MUL)
            p.grad = Tensor.randn_on(shape, 12 + 100 * l + k, dev).raw_binary(Tensor.scalar_on(1e-3, dev), op.MUL)
            params.append(p)
    acts = [Tensor.randn_on([batch, width], 500 + l, dev) for l in range(layers - 1)]
    target = Tensor.randn_on([batch, width], 600, dev)
    opt = SGD(params, 0.01)

    def step():
        ys = [a.raw_unary(op.RELU) for a in acts]                      # ReLU forward, 11 times
        last = ys[-1].detach().requires_grad_()
        loss = mse_loss(last, target)                                  # SUB, MUL, SUM_AXIS, DIV
        loss.backward()                                                # gradient of the mean back to `last`
        g = last.grad
        for a in acts:                                                 # ReLU backward: g * STEP(x)
            g_in = g.relu_grad(a)
        opt.step()                                                     # AXPY per parameter tensor
        return loss, g_in

    return step


def config4(dev: Device, transposed: bool, B: int = 64, R: int = 2048, Cn: int = 2048):
    m1 = Tensor.randn_on([B, 1, Cn], 22, dev)
    m2 = Tensor.from_numpy(synth.softmax_mask(R), dev)  # -1e4 * Bernoulli(0.1) from seed 22
    X = Tensor.randn_on([B, Cn, R] if transposed else [B, R, Cn], 21, dev).raw_binary(Tensor.scalar_on(2.0, dev), op.MUL)
    shape = [B, R, Cn]

    def step():
        if transposed:  # X stored [B, Cn, R], read as [B, R, Cn] through strides (R*Cn, 1, R)
            Y1 = run_op(dev, op.ADD, [0], [Operand(X, shape, [R * Cn, 1, R]), Operand(m1, shape, broadcast_strides(m1.shape, shape))], shape)
        else:
            Y1 = X + m1
        Y = Y1 + m2
        M = Y.max_dim(2, keepdim=True)
        E = Y.sub_exp(M)  # SUB then EXP unless the device uses the fused op
        S = E.sum_dim(2, keepdim=True)
        return E / S

    return step


def split_layers_of(layers: int, rank: int, world: int) -> range:
    """The layers ``rank`` owns when whole layers are dealt to ranks in contiguous blocks (the reference's
    layer-split placement, crates/core/src/strategy.rs:269-326)."""
    from pytorches_b200.shard import split_layers

    lo, count = split_layers(layers, rank, world)
    return range(lo, lo + count)


def config3_sharded(dev: Device, rank: int, world: int, layers: int = 12, width: int = 8192, batch: int = 32):
    """Config 3 with its layers dealt to ``world`` ranks: a rank holds, activates and updates only the
    layers it owns (no exchange: the config is the elementwise part of the step); the loss belongs to
    the owner of the last layer. With one rank this is ``config3``."""
    own = split_layers_of(layers, rank, world)
    params = []
    for l in own:
        for shape, k in (([width, width], 0), ([width], 1)):
            p = Tensor.randn_on(shape, 11 + 100 * l + k, dev).raw_binary(Tensor.scalar_on(0.02, dev), op.MUL)
            p.grad = Tensor.randn_on(shape, 12 + 100 * l + k, dev).raw_binary(Tensor.scalar_on(1e-3, dev), op.MUL)
            params.append(p)
    acts = {l: Tensor.randn_on([batch, width], 500 + l, dev) for l in own if l < layers - 1}  # a ReLU follows every layer but the last
    last = layers - 1 in own
    seed_act = Tensor.randn_on([batch, width], 500 + layers - 2, dev) if last and layers - 2 not in acts else None
    target = Tensor.randn_on([batch, width], 600, dev) if last else None
    g_next = None if last else Tensor.randn_on([batch, width], 700 + rank, dev)  # the gradient that arrives from the next rank's layers
    opt = SGD(params, 0.01)

    def step():
        ys = {l: a.raw_unary(op.RELU) for l, a in acts.items()}
        loss = g = None
        if last:
            y = ys.get(layers - 2)
            if y is None:
                y = seed_act.raw_unary(op.RELU)
            pred = y.detach().requires_grad_()
            loss = mse_loss(pred, target)
            loss.backward()
            g = pred.grad
        else:
            g = g_next
        g_in = None
        for a in acts.values():
            g_in = g.relu_grad(a)
        opt.step()
        return loss, g_in, params

    return step


def measure(name: str, make, plugin: Plugin, device_index: int, iters: int, stream=None, fused: bool = False, python: bool = False):
    """One config on one device. The step runs once through the Python mirror of the reference core with
    a recorder in between; its calls (alloc, execute, free: 'allocation inside the timed region, as the
    core would run it') are then replayed by native code and timed with CUDA events, unless ``python``
    keeps the Python mirror in the loop. Also reports what the host needs to enqueue one call."""
    from pytorches_b200.replay import Recorder, algorithmic_bytes

    recorder = Recorder(plugin)
    dev = Device(recorder, device_index, fused=fused)
    step = make(dev)
    step()  # warm-up, also fills the allocator's cache
    dev.synchronize()
    recorder.start()
    keep = step()
    rec = recorder.finish(device_index)
    del keep
    nbytes, nops = algorithmic_bytes(rec), rec.executes
    dev.synchronize()
    run = step if python or stream is None else (lambda: rec.run(1))
    for _ in range(3):
        run()
    dev.synchronize()
    times, host = [], []
    if stream is not None:
        import torch

        for _ in range(iters):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(stream)
            t = time.perf_counter()
            run()
            host.append((time.perf_counter() - t) * 1e3)
            b.record(stream)
            dev.synchronize()
            torch.cuda.synchronize()
            times.append(a.elapsed_time(b))
    else:
        for _ in range(iters):
            t = time.perf_counter()
            run()
            dev.synchronize()
            times.append((time.perf_counter() - t) * 1e3)
    ms = statistics.median(times)
    out = {"config": name, "plugin": plugin.name, "ops_per_step": nops, "algorithmic_bytes": nbytes, "ms": round(ms, 4),
           "GB/s": round(nbytes / (ms * 1e-3) / 1e9, 1), "driven_by": "Python mirror of the core" if python or stream is None else "recorded calls replayed natively"}
    if host:
        out["host_enqueue_ms"] = round(statistics.median(host), 4)
        out["host_us_per_call"] = round(statistics.median(host) * 1e3 / max(rec.n, 1), 2)
        out["calls_per_step"] = rec.n
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", default="1,3,4,4t")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--device", type=int, default=0)
    ap.add_argument("--peak", type=float, default=6454.6)
    ap.add_argument("--python", action="store_true", help="also time each config with the Python mirror of the core issuing the calls")
    ap.add_argument("--fused", action="store_true",
                    help="also run each config with the optional fused ops (RELU_GRAD, ADD_RELU, SUB_EXP) in place of the reference's "
                         "two-op sequences; same results, fewer bytes")
    args = ap.parse_args()
    world, rank = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0"))
    if world > 1:
        args.device = int(os.environ.get("LOCAL_RANK", "0"))
    makers = {"1": ("config 1: bias+relu+scale, row sums, backward", config1),
              "3": ("config 3: MLP elementwise part + SGD over 805M parameters", lambda d: config3_sharded(d, rank, world)),
              "4": ("config 4: softmax from primitives, contiguous X", lambda d: config4(d, False)),
              "4t": ("config 4: softmax from primitives, transposed X", lambda d: config4(d, True))}
    import torch

    plugin = pytorches_b200.load_plugin()
    if plugin.device_count() <= args.device:
        raise SystemExit("no CUDA device: the B200 plugin has no fallback")
    get_stream = plugin.lib.pytorches_b200_stream
    get_stream.restype, get_stream.argtypes = ctypes.c_void_p, [ctypes.c_uint32]
    torch.cuda.set_device(args.device)
    stream = torch.cuda.ExternalStream(get_stream(args.device), device=torch.device("cuda", args.device))
    if world > 1:
        import torch.distributed as dist

        from pytorches_b200.shard import nccl_options

        dist.init_process_group("nccl", device_id=torch.device("cuda", args.device), pg_options=nccl_options())

    def across_ranks(r):
        """Layer-sharded config 3: the step takes as long as the slowest rank; bytes and ops add up."""
        if world == 1:
            return r
        t = torch.tensor([r["ms"], float(r["algorithmic_bytes"]), float(r["ops_per_step"])], dtype=torch.float64, device=f"cuda:{args.device}")
        slow = t.clone()
        dist.all_reduce(slow, op=dist.ReduceOp.MAX)
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        r = dict(r, ms=round(float(slow[0]), 4), algorithmic_bytes=int(t[1]), ops_per_step=int(t[2]))
        r["GB/s"] = round(r["algorithmic_bytes"] / (r["ms"] * 1e-3) / 1e9, 1)
        layers = 12
        r["gpus"] = world
        r["ideal_speedup_over_1_gpu"] = round(layers / max(len(split_layers_of(layers, k, world)) for k in range(world)), 2)
        return r

    try:
        for key in args.config.split(","):
            if world > 1 and key != "3":
                continue  # only config 3 is sharded by layer; the others shard by rows (opbench, bench.py)
            title, make = makers[key]
            variants = [(title, False, False)]
            if args.python:
                variants.append((title + " [Python-driven]", False, True))
            if args.fused:
                variants.append((title + " [fused ops]", True, False))
            base = None
            for label, fused, python in variants:
                r = across_ranks(measure(label, make, plugin, args.device, args.iters, stream, fused=fused, python=python))
                r["frac_of_peak"] = round(r["GB/s"] / (args.peak * world), 4)
                r["frac_of_8TBps"] = round(r["GB/s"] / (8000.0 * world), 4)
                if base is None:
                    base = r
                elif fused:
                    r["speedup_vs_reference_sequence"] = round(base["ms"] / r["ms"], 3)
                    r["GB/s_of_reference_sequence_bytes"] = round(base["algorithmic_bytes"] / (r["ms"] * 1e-3) / 1e9, 1)
                if rank == 0:
                    print(json.dumps(r))
                    sys.stdout.flush()
    finally:
        if world > 1:
            dist.destroy_process_group()


if __name__ == "__main__":
    main()
