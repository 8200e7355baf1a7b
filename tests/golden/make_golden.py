"""Generates tests/golden/cpuref_vectors.npz: outputs of the CPU oracle on fixed seeded inputs.

The reference stores no fixture files (its test vectors come from an in-test LCG, restated in
tests/harness.py), so these are not reference outputs: they freeze what the oracle computes TODAY,
on an AVX2+FMA host, for inputs whose results do not depend on the C library (whole 8-lane vectors for
exp/log/tanh, exact arithmetic elsewhere). A later change of compiler flags or of the restatement
that moves a single bit shows up as a diff against this file, on the CPU and on the GPU.

Run from the repository root:  python tests/golden/make_golden.py
"""

import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

from conformance import edge_values  # noqa: E402
from harness import Buf, exec_op, lcg_data  # noqa: E402
from pytorches_b200.abi import Plugin, contiguous_strides, op  # noqa: E402


def cases():
    """(name, op code, ints, [(host array, shape, strides)], output shape)."""
    x = edge_values()
    x = np.concatenate([x, np.zeros((-x.size) % 8, dtype=np.float32)])
    n = x.size
    out = [("exp_edge", op.EXP, [0], [(x, (n,), (1,))], (n,)), ("log_edge", op.LOG, [0], [(x, (n,), (1,))], (n,)),
           ("tanh_edge", op.TANH, [0], [(x, (n,), (1,))], (n,))]
    a, b = lcg_data(4096, 5), lcg_data(4096, 6) + np.float32(1.5)
    for name, code in (("add", op.ADD), ("sub", op.SUB), ("mul", op.MUL), ("div", op.DIV)):
        out.append((f"{name}_bcast", code, [0], [(a, (64, 64), (64, 1)), (b, (64, 64), (0, 1))], (64, 64)))
    s = lcg_data(65536 * 3 + 77, 7)
    out.append(("sum_blocks", op.SUM_AXIS, [0], [(s, (s.size,), (1,))], ()))
    m = lcg_data(300 * 64, 8)
    out.append(("sum_cols", op.SUM_AXIS, [0], [(m, (300, 64), (64, 1))], (64,)))
    out.append(("sum_rows", op.SUM_AXIS, [1], [(m, (300, 64), (64, 1))], (300,)))
    out.append(("axpy", op.AXPY, [int(np.float32(-0.01).view(np.uint32))], [(a, (4096,), (1,)), (b, (4096,), (1,))], (4096,)))
    out.append(("relu", op.RELU, [0], [(a, (4096,), (1,))], (4096,)))
    return out


def run(plugin):
    res = {}
    for name, code, ints, ins, oshape in cases():
        bufs = [(Buf(plugin, h), sh, st) for (h, sh, st) in ins]
        o = Buf.empty(plugin, int(np.prod(oshape)) if len(oshape) else 1)
        assert exec_op(plugin, code, ints, bufs, o, oshape) == 0, plugin.last_error()
        res[name] = o.get()
    return res


if __name__ == "__main__":
    oracle = Plugin(os.path.join(ROOT, "oracle", "_build", "pytorches_plugin_cpuref.so"))
    np.savez_compressed(os.path.join(ROOT, "tests", "golden", "cpuref_vectors.npz"), **run(oracle))
    print("wrote", len(cases()), "vectors")
