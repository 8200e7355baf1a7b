"""Seeded random layouts: shapes of 1 to 5 dims whose operands are contiguous, broadcast along a random
subset of dims (stride 0), or stored in a permuted order (transposed views), in any mix.

The hand-picked cases of the parity tests name the layouts the reference's tests use; these go
looking for the ones nobody thought of, since the choice between the flat, row, tile and gather
kernels (and the coalescing in front of it, plugins/cpu/src/ew.rs:22-43) depends on exactly these
details. CPU run: the oracle against numpy. GPU run: the B200 plugin against the oracle.
"""

import numpy as np
import pytest

from harness import Buf, assert_bit_equal, exec_op, lcg_data, ulp_distance
from pytorches_b200 import abi
from pytorches_b200.abi import op


def random_case(rng):
    """(shape, strides of a, strides of b), strides in elements over the output's shape."""
    nd = int(rng.integers(1, 6))
    budget = int(rng.choice([200, 5_000, 70_000, 300_000]))
    shape = []
    for _ in range(nd):
        hi = max(2, int(round(budget ** (1.0 / nd) * 2)))
        shape.append(int(rng.choice([1, int(rng.integers(1, hi)), int(rng.integers(1, hi)), int(rng.choice([4, 8, 32, 64, 128]))])))
    while int(np.prod(shape)) > 400_000:
        shape[int(np.argmax(shape))] //= 2

    def operand():
        kind = rng.choice(["dense", "broadcast", "permuted", "both"])
        stored = list(shape)
        if kind in ("broadcast", "both"):
            for d in range(nd):
                if rng.random() < 0.4:
                    stored[d] = 1
        order = list(range(nd))
        if kind in ("permuted", "both"):
            rng.shuffle(order)
        strides, acc = [0] * nd, 1
        for d in reversed(order):  # order[-1] is the fastest dim in storage
            if stored[d] == 1 and shape[d] != 1:
                strides[d] = 0  # broadcast along d
            else:
                strides[d] = acc
                acc *= stored[d]
        return tuple(strides)

    return tuple(shape), operand(), operand()


def storage(shape, strides, seed, scale=1.0):
    span = 1 + sum((s - 1) * st for s, st in zip(shape, strides))
    return (lcg_data(span, seed) * np.float32(scale)).astype(np.float32)


def view(store, shape, strides):
    return np.lib.stride_tricks.as_strided(store, shape=shape, strides=tuple(4 * s for s in strides))


def run(p, code, ins, shape):
    n = int(np.prod(shape))
    bufs = [(Buf(p, h), shape, st) for h, st in ins]
    out = Buf.empty(p, n)
    assert exec_op(p, code, [0], bufs, out, shape) == abi.STATUS_OK, f"{p.name}: {p.last_error()}"
    return out.get()


CASES = [random_case(np.random.default_rng(1000 + i)) for i in range(160)]


@pytest.mark.parametrize("k", range(0, 60))
def test_oracle_matches_numpy_on_random_layouts(oracle, k):
    shape, sa, sb = CASES[k]
    if int(np.prod(shape)) == 0:
        pytest.skip("empty")
    a, b = storage(shape, sa, 2 * k + 1), storage(shape, sb, 2 * k + 2) + np.float32(1.5)
    for code, fn in ((op.ADD, np.add), (op.MUL, np.multiply), (op.DIV, np.divide), (op.SUB, np.subtract)):
        got = run(oracle, code, [(a, sa), (b, sb)], shape)
        assert_bit_equal(f"{code} {shape} {sa} {sb}", got, fn(view(a, shape, sa), view(b, shape, sb)).astype(np.float32).reshape(-1))
    got = run(oracle, op.RELU, [(a, sa)], shape)
    assert_bit_equal(f"relu {shape} {sa}", got, np.maximum(view(a, shape, sa), np.float32(0)).reshape(-1), zero_sign_matters=False)


@pytest.mark.gpu
@pytest.mark.parametrize("k", range(len(CASES)))
def test_b200_matches_oracle_on_random_layouts(oracle, b200, k):
    shape, sa, sb = CASES[k]
    if int(np.prod(shape)) == 0:
        pytest.skip("empty")
    a, b = storage(shape, sa, 2 * k + 1), storage(shape, sb, 2 * k + 2)
    what = f"{shape} {sa} {sb}"
    for code in (op.ADD, op.MUL, op.DIV, op.RELU_GRAD, op.ADD_RELU):
        assert_bit_equal(f"{code} {what}", run(b200, code, [(a, sa), (b, sb)], shape), run(oracle, code, [(a, sa), (b, sb)], shape))
    for code in (op.NEG, op.RELU, op.STEP, op.COPY):
        assert_bit_equal(f"{code} {what}", run(b200, code, [(a, sa)], shape), run(oracle, code, [(a, sa)], shape), zero_sign_matters=code != op.RELU)
    a9 = storage(shape, sa, 2 * k + 1, 9.0)
    for code in (op.EXP, op.TANH):  # the polynomial elements are bit-equal, the libm ones within 2 ulp
        got, want = run(b200, code, [(a9, sa)], shape), run(oracle, code, [(a9, sa)], shape)
        assert int(ulp_distance(got, want).max()) <= 2, f"{code} {what}"
    got, want = run(b200, op.SUB_EXP, [(a9, sa), (b, sb)], shape), run(oracle, op.SUB_EXP, [(a9, sa), (b, sb)], shape)
    assert int(ulp_distance(got, want).max()) <= 2, f"SUB_EXP {what}"
    body = got.size - got.size % 8
    assert_bit_equal(f"SUB_EXP body {what}", got[:body], want[:body])
