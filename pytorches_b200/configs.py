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

Usage:  python -m pytorches_b200.configs [--config 1,3,4] [--iters 10] [--cpu]   (--cpu times the CPU oracle too)
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
from pytorches_b200.abi import Plugin, op
from pytorches_b200.core import SGD, Device, Operand, Tensor, broadcast_strides, mse_loss, run_op


class CountingPlugin:
    """Wraps a plugin and adds up the algorithmic bytes and launches of every ``execute`` it forwards."""

    def __init__(self, plugin: Plugin):
        self._p = plugin
        self.bytes = 0
        self.ops = 0

    def __getattr__(self, name):
        return getattr(self._p, name)

    @staticmethod
    def _stored(arg) -> int:
        n = 1
        for size, stride in zip(arg.shape, arg.strides):
            if stride != 0:
                n *= size
        return n * (8 if arg.dtype == 1 else 4)

    def execute(self, device, code, ints, inputs, outputs):
        seen = set()
        for a in inputs:
            if a.data not in seen:  # d*d reads d once
                seen.add(a.data)
                self.bytes += self._stored(a)
        for o in outputs:
            self.bytes += math.prod(o.shape) * (8 if o.dtype == 1 else 4)
        self.ops += 1
        return self._p.execute(device, code, ints, inputs, outputs)


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
    m2_host = np.where(np.random.default_rng(22).random(R) < 0.1, np.float32(-1e4), np.float32(0.0)).astype(np.float32).reshape(1, R, 1)
    m2 = Tensor.from_numpy(m2_host, dev)
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


def measure(name: str, make, plugin: Plugin, device_index: int, iters: int, stream=None, fused: bool = False):
    counting = CountingPlugin(plugin)
    dev = Device(counting, device_index, fused=fused)
    step = make(dev)
    step()  # warm-up, also fills the allocator's cache
    dev.synchronize()
    counting.bytes = counting.ops = 0
    step()
    nbytes, nops = counting.bytes, counting.ops
    dev.synchronize()
    times = []
    if stream is not None:
        import torch

        for _ in range(iters):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(stream)
            step()
            b.record(stream)
            dev.synchronize()
            torch.cuda.synchronize()
            times.append(a.elapsed_time(b))
    else:
        for _ in range(iters):
            t = time.perf_counter()
            step()
            dev.synchronize()
            times.append((time.perf_counter() - t) * 1e3)
    ms = statistics.median(times)
    return {"config": name, "plugin": plugin.name, "ops_per_step": nops, "algorithmic_bytes": nbytes, "ms": round(ms, 4),
            "GB/s": round(nbytes / (ms * 1e-3) / 1e9, 1)}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", default="1,3,4,4t")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--device", type=int, default=0)
    ap.add_argument("--cpu", action="store_true", help="also time the CPU oracle (test infrastructure) on the same configs")
    ap.add_argument("--peak", type=float, default=6454.6)
    ap.add_argument("--fused", action="store_true",
                    help="also run each config with the optional fused ops (RELU_GRAD, ADD_RELU, SUB_EXP) in place of the reference's "
                         "two-op sequences; same results, fewer bytes")
    args = ap.parse_args()
    makers = {"1": ("config 1: bias+relu+scale, row sums, backward", config1),
              "3": ("config 3: MLP elementwise part + SGD over 805M parameters", config3),
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
    oracle = None
    if args.cpu:
        root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
        oracle = Plugin(os.path.join(root, "oracle", "_build", "pytorches_plugin_cpuref.so"))
    for key in args.config.split(","):
        title, make = makers[key]
        r = measure(title, make, plugin, args.device, args.iters, stream)
        r["frac_of_peak"] = round(r["GB/s"] / args.peak, 4)
        r["frac_of_8TBps"] = round(r["GB/s"] / 8000.0, 4)
        if oracle is not None:
            c = measure(title, make, oracle, 0, max(2, args.iters // 4))
            r["cpu_oracle_ms"], r["cpu_oracle_GB/s"], r["cpu_threads"] = c["ms"], c["GB/s"], os.cpu_count()
        print(json.dumps(r))
        sys.stdout.flush()
        if args.fused:
            f = measure(title + " [fused ops]", make, plugin, args.device, args.iters, stream, fused=True)
            f["speedup_vs_reference_sequence"] = round(r["ms"] / f["ms"], 3)
            f["GB/s_of_reference_sequence_bytes"] = round(r["algorithmic_bytes"] / (f["ms"] * 1e-3) / 1e9, 1)
            print(json.dumps(f))
            sys.stdout.flush()


if __name__ == "__main__":
    main()
