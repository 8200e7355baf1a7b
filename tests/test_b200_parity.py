"""Parity of the B200 plugin with the CPU oracle on identical seeded inputs (GPU run).

Both plugins are driven through the same C ABI with the same host data. Bars:
  * ADD/SUB/MUL/DIV/NEG/RELU/STEP/COPY/AXPY/FILL: bit-exact (RELU: +0 and -0 compare equal);
  * SUM_AXIS: bit-exact as well, because the kernels keep the reference's association order
    (the required bar is only a relative 1e-5*log2(n));
  * EXP/LOG/TANH: bit-exact wherever the reference runs its vector polynomial, and within 2 ulp on the
    few elements it hands to libm (the last len mod 8 of a row);
  * RAND_NORMAL: the integer hash is exact; ln/cos differ by library, so 1e-5 absolute like the
    reference's golden-value test (crates/core/src/lib.rs:929-937);
  * MAX/ARGMAX: bit-exact / index-exact.
"""

import math
import struct

import numpy as np
import pytest

from harness import Buf, assert_bit_equal, exec_op, lcg_data, ulp_distance
from pytorches_b200 import abi
from pytorches_b200.abi import DTYPE_I64, contiguous_strides, op
from pytorches_b200 import synth
from pytorches_b200.core import SGD, Device, Tensor, mse_loss

pytestmark = pytest.mark.gpu


def f32_bits(v):
    return struct.unpack("<I", struct.pack("<f", v))[0]


def both(oracle, b200, code, ints, ins, oshape, out_dtype=abi.DTYPE_F32):
    """Runs one op on both plugins. ``ins`` = [(host array, shape, strides)]; returns (got, want)."""
    n = int(np.prod(oshape)) if len(oshape) else 1
    res = []
    for p in (b200, oracle):
        bufs = [(Buf(p, h), sh, st) for (h, sh, st) in ins]
        out = Buf.empty(p, n, dtype=np.int64 if out_dtype == DTYPE_I64 else np.float32)
        st = exec_op(p, code, ints, bufs, out, oshape, out_dtype)
        assert st == abi.STATUS_OK, f"{p.name}: {p.last_error()}"
        res.append(out.get())
    return res[0], res[1]


# shape, strides of operand A, strides of operand B (both over the output's shape)
BROADCAST_CASES = [
    ((1000,), (1,), (1,)),
    ((1000,), (1,), (0,)),
    ((1000,), (0,), (1,)),
    ((4099,), (1,), (1,)),                       # ragged tail
    ((37, 91), (91, 1), (0, 1)),                 # row vector, odd sizes (scalar path)
    ((64, 128), (128, 1), (0, 1)),               # row vector, float4 path
    ((64, 128), (128, 1), (1, 0)),               # column vector
    ((64, 128), (0, 1), (1, 0)),                 # outer product
    ((64, 128), (0, 0), (128, 1)),               # scalar
    ((8, 16, 32), (512, 32, 1), (32, 0, 1)),     # [B,1,N] broadcast on the middle dim
    ((8, 16, 32), (512, 32, 1), (0, 1, 0)),      # [1,M,1]
    ((8, 16, 32), (512, 32, 1), (16, 1, 0)),     # [B,M,1] broadcast on the last dim
    ((8, 16, 32), (512, 1, 16), (32, 0, 1)),     # transposed view on the last two dims
    ((5, 7, 9), (63, 1, 7), (63, 9, 1)),         # transposed, odd sizes
    ((33, 65), (1, 33), (65, 1)),                # plain 2-D transpose
    ((33, 65), (1, 33), (1, 33)),                # both transposed
    ((6, 5, 4, 3), (60, 12, 3, 1), (0, 12, 0, 1)),
    ((3, 4, 5, 6, 7), (840, 210, 42, 7, 1), (0, 0, 42, 0, 1)),
    ((2, 3, 4), (1, 2, 6), (12, 4, 1)),          # fully permuted: gather path
    ((64, 128), (1, 64), (128, 1)),              # transposed, 128-bit friendly sizes (wide tile kernel)
    ((128, 64), (1, 128), (1, 128)),             # both transposed, wide tiles
    ((8, 64, 128), (8192, 1, 64), (128, 0, 1)),  # batched transposed + broadcast row operand
    ((8, 100, 132), (13200, 1, 100), (0, 1, 0)), # transposed with ragged 64x64 tiles, scalar-mode partner
    ((3, 5, 64, 68), (21760, 4352, 1, 64), (0, 4352, 68, 1)),  # two batch dims around a transposed pair
    ((300_000,), (1,), (1,)),
    ((1 << 20,), (1,), (1,)),
    ((1024, 1024), (1024, 1), (0, 1)),
    ((1024, 1024), (1024, 1), (1, 0)),
]


def storage_for(shape, strides, seed, shift=0.0):
    span = 1 + sum((s - 1) * st for s, st in zip(shape, strides))
    return lcg_data(span, seed) + np.float32(shift)


@pytest.mark.parametrize("shape,sa,sb", BROADCAST_CASES)
def test_binary_ops_bit_exact(oracle, b200, shape, sa, sb):
    a = storage_for(shape, sa, 5)
    b = storage_for(shape, sb, 6, 1.5)
    for code in (op.ADD, op.SUB, op.MUL, op.DIV):
        got, want = both(oracle, b200, code, [0], [(a, shape, sa), (b, shape, sb)], shape)
        assert_bit_equal(f"binary {code} {shape} {sa} {sb}", got, want)


@pytest.mark.parametrize("shape,sa,sb", BROADCAST_CASES + [((7,), (1,), (1,)), ((65543,), (1,), (0,)), ((5, 13), (13, 1), (1, 0))])
def test_fused_ops_bit_exact(oracle, b200, shape, sa, sb):
    """RELU_GRAD, ADD_RELU, SUB_EXP: the oracle computes them as their two-op sequences; every layout the
    binary kernels serve must give those bits, the libm-computed last (n mod 8) elements of SUB_EXP within 2 ulp."""
    a = storage_for(shape, sa, 5)
    b = storage_for(shape, sb, 6)  # both zero-centred: relu and step see both signs
    for code in (op.RELU_GRAD, op.ADD_RELU):
        got, want = both(oracle, b200, code, [0], [(a, shape, sa), (b, shape, sb)], shape)
        assert_bit_equal(f"fused {code} {shape} {sa} {sb}", got, want)
    a20 = a * np.float32(20.0)
    got, want = both(oracle, b200, op.SUB_EXP, [0], [(a20, shape, sa), (b, shape, sb)], shape)
    n = got.size
    body = n - n % 8
    assert_bit_equal(f"SUB_EXP body {shape} {sa} {sb}", got[:body], want[:body])
    assert int(ulp_distance(got[body:], want[body:]).max(initial=0)) <= 2


def test_fused_ops_special_values_bit_exact(oracle, b200):
    specials = np.array([0.0, -0.0, 1e-45, -1e-45, 1e-38, 1.0, -1.0, 3.4e38, -3.4e38, np.inf, -np.inf, np.nan, 1e-20, 1e20, 88.0, -104.0],
                        dtype=np.float32)
    a = np.repeat(specials, specials.size)
    b = np.tile(specials, specials.size)
    sh = (a.size,)  # 256 elements: no libm tail
    for code in (op.RELU_GRAD, op.ADD_RELU, op.SUB_EXP):
        got, want = both(oracle, b200, code, [0], [(a, sh, (1,)), (b, sh, (1,))], sh)
        assert_bit_equal(f"fused {code} specials", got, want, zero_sign_matters=code != op.ADD_RELU)


def test_binary_special_values_bit_exact(oracle, b200):
    specials = np.array([0.0, -0.0, 1e-45, -1e-45, 1e-38, 1.0, -1.0, 3.4e38, -3.4e38, np.inf, -np.inf, np.nan, 1e-20, 1e20], dtype=np.float32)
    a = np.repeat(specials, specials.size)
    b = np.tile(specials, specials.size)
    sh = (a.size,)
    for code in (op.ADD, op.SUB, op.MUL, op.DIV):
        got, want = both(oracle, b200, code, [0], [(a, sh, (1,)), (b, sh, (1,))], sh)
        assert_bit_equal(f"binary {code} specials", got, want)


UNARY_SHAPES = [((256, 128), (1, 256)), ((4, 64, 72), (4608, 1, 64)), ((1000,), (1,)), ((4099,), (1,)), ((7,), (1,)), ((300_001,), (1,)), ((33, 65), (1, 33)), ((16, 8), (0, 1)), ((16, 8), (1, 0))]


@pytest.mark.parametrize("shape,st", UNARY_SHAPES)
def test_exact_unary_ops(oracle, b200, shape, st):
    x = storage_for(shape, st, 12)
    x[:: 7] = 0.0
    x[3:: 11] = -0.0
    for code in (op.NEG, op.RELU, op.STEP, op.COPY):
        got, want = both(oracle, b200, code, [0], [(x, shape, st)], shape)
        assert_bit_equal(f"unary {code} {shape} {st}", got, want, zero_sign_matters=(code != op.RELU))


def transcendental_inputs(n, seed):
    x = lcg_data(n, seed)
    return {op.EXP: x * np.float32(20.0), op.LOG: np.abs(x) * np.float32(50.0) + np.float32(1e-6), op.TANH: x * np.float32(9.0)}


@pytest.mark.parametrize("n", [8, 64, 1003, 65536, 65536 * 3 + 5, 1 << 20])
def test_exp_log_tanh_match_the_vector_polynomials(oracle, b200, n):
    """Contiguous input: the reference runs the polynomial on the first n - n%8 elements (bit-exact
    here) and libm on the last n%8 (within 2 ulp here)."""
    for code, x in transcendental_inputs(n, 13).items():
        got, want = both(oracle, b200, code, [0], [(x, (n,), (1,))], (n,))
        body = n - n % 8
        assert_bit_equal(f"op {code} n={n} body", got[:body], want[:body])
        assert ulp_distance(got[body:], want[body:]).max(initial=0) <= 2, f"op {code} n={n} tail"


def test_exp_log_tanh_edge_values(oracle, b200):
    from conformance import edge_values

    x = edge_values()
    x = np.concatenate([x, np.zeros((-x.size) % 8, dtype=np.float32)])  # whole vectors only: polynomial everywhere
    for code in (op.EXP, op.LOG, op.TANH):
        got, want = both(oracle, b200, code, [0], [(x, (x.size,), (1,))], (x.size,))
        assert_bit_equal(f"op {code} edge values", got, want)


@pytest.mark.parametrize("shape,st", [((33, 65), (1, 33)), ((128, 320), (1, 128)), ((2, 64, 300), (19200, 1, 64))])
def test_exp_log_tanh_strided_within_2ulp(oracle, b200, shape, st):
    """Strided inputs reach the reference's gather path, where the libm / polynomial split falls every
    256 gathered elements: the bar there is 2 ulp everywhere, and bit-equality on most elements."""
    n = int(np.prod(shape))
    for code, x in transcendental_inputs(n, 14).items():
        got, want = both(oracle, b200, code, [0], [(x, shape, st)], shape)
        d = ulp_distance(got, want)
        assert d.max() <= 2
        assert (d == 0).mean() > 0.9


@pytest.mark.parametrize("n", [1, 7, 8, 33, 4097, 65536, 65543, 300_000, (1 << 20) + 3])
def test_axpy_bit_exact(oracle, b200, n):
    """FMA body, unfused last n%8 (plugins/cpu/src/ew.rs:316-329), in place and out of place."""
    a, b = lcg_data(n, 8), lcg_data(n, 9)
    alpha = f32_bits(-0.01)
    got, want = both(oracle, b200, op.AXPY, [alpha], [(a, (n,), (1,)), (b, (n,), (1,))], (n,))
    assert_bit_equal(f"axpy n={n}", got, want)
    res = []
    for p in (b200, oracle):  # in place: the output is the first input's buffer
        A, B = Buf(p, a), Buf(p, b)
        assert exec_op(p, op.AXPY, [alpha], [(A, (n,), (1,)), (B, (n,), (1,))], A, (n,)) == abi.STATUS_OK
        res.append(A.get())
    assert_bit_equal(f"axpy in place n={n}", res[0], res[1])


SUM_CASES = [(1000,), (33, 17), (5, 4, 3), (70_001,), (3, 200_000), (100_000, 3), (2, 600, 5), (4, 4096, 70), (1, 1), (64, 4096),
             (300, 64), (2, 1000, 36), (1, 129, 32), (5000, 128), (31,), (32,), (33,), (65536,), (65537,), (65536 * 5 + 77,), (4096, 4096), (1 << 22,), (128, 2048),
             # column sums through the transposing kernel: ragged tiles, ragged column groups, several slabs, many tiles
             (1000, 96), (3, 257, 160), (520, 40), (16384, 256), (127, 64), (128, 32), (129, 4100), (2, 385, 36), (40_000, 32)]


@pytest.mark.parametrize("shape", SUM_CASES)
def test_sum_axis_bit_exact(oracle, b200, shape):
    n = int(np.prod(shape))
    x = lcg_data(n, 7)
    for axis in range(len(shape)):
        oshape = tuple(s for i, s in enumerate(shape) if i != axis)
        got, want = both(oracle, b200, op.SUM_AXIS, [axis], [(x, shape, contiguous_strides(shape))], oshape)
        assert_bit_equal(f"sum {shape} axis {axis}", got, want)
        # and the bar the contract actually asks for, against an f64 sum
        ref = x.reshape(shape).astype(np.float64).sum(axis=axis).reshape(-1)
        scale = np.abs(x.reshape(shape).astype(np.float64)).sum(axis=axis).reshape(-1)
        tol = 1e-5 * max(math.log2(max(shape[axis], 2)), 1.0)
        assert np.all(np.abs(got - ref) <= tol * np.maximum(scale, 1e-30))


@pytest.mark.parametrize("shape", [(1000,), (70_001,), (3, 200_000), (100_000, 3), (2, 600, 5), (64, 4096), (1 << 22,), (128, 2048), (5, 16385),
                                   ((1 << 22) + 65536 * 3 + 4101,), ((1 << 23) + 7,)])
def test_max_argmax_match_oracle(oracle, b200, shape):
    n = int(np.prod(shape))
    x = (np.round(lcg_data(n, 11) * 64) / 64).astype(np.float32)  # plenty of ties
    for axis in range(len(shape)):
        oshape = tuple(s for i, s in enumerate(shape) if i != axis)
        ins = [(x, shape, contiguous_strides(shape))]
        got, want = both(oracle, b200, op.MAX_AXIS, [axis], ins, oshape)
        assert_bit_equal(f"max {shape} axis {axis}", got, want, zero_sign_matters=False)
        got, want = both(oracle, b200, op.ARGMAX_AXIS, [axis], ins, oshape, DTYPE_I64)
        assert np.array_equal(got, want), f"argmax {shape} axis {axis}"


def test_argmax_all_minus_inf_and_nan_first(oracle, b200):
    for n in (5, 4096, 70_000, (1 << 22) + 65536 + 12):  # the last one takes the staged kernel for one long row
        x = np.full(n, -np.inf, dtype=np.float32)
        got, want = both(oracle, b200, op.ARGMAX_AXIS, [0], [(x, (n,), (1,))], (), DTYPE_I64)
        assert got[0] == want[0] == 0
        x = lcg_data(n, 3)
        x[n // 2] = np.nan
        x[n - 1] = np.nan
        got, want = both(oracle, b200, op.ARGMAX_AXIS, [0], [(x, (n,), (1,))], (), DTYPE_I64)
        assert got[0] == want[0] == n // 2
        got, want = both(oracle, b200, op.MAX_AXIS, [0], [(x, (n,), (1,))], ())
        assert np.isnan(got[0]) and np.isnan(want[0])


def test_fill_and_randn(oracle, b200):
    for n in (1, 5, 4099, 1 << 20):
        got, want = both(oracle, b200, op.FILL, [f32_bits(-2.5)], [], (n,))
        assert_bit_equal(f"fill n={n}", got, want)
        got, want = both(oracle, b200, op.RAND_NORMAL, [1234], [], (n,))
        assert np.max(np.abs(got - want)) <= 1e-5, f"randn n={n}: {np.max(np.abs(got - want))}"
        # RAND_UNIFORM (appended): hash, one multiply, one add; exact on both sides and equal to the numpy generator
        for lo, hi, first in ((-1.0, 1.0, 0), (0.5, 2.0, 1 << 33)):
            ints = [31, f32_bits(lo), f32_bits(hi - lo), first]
            got, want = both(oracle, b200, op.RAND_UNIFORM, ints, [], (n,))
            assert_bit_equal(f"rand_uniform n={n}", got, want)
            assert_bit_equal(f"rand_uniform n={n} vs numpy", got, synth.uniform(n, 31, lo, hi, first))


# ---- the benchmark configurations, at sizes the oracle finishes in seconds, through the mini-core ----

def run_on(plugin, fn):
    dev = Device(plugin, 0)
    return [t if isinstance(t, np.ndarray) else t.numpy() for t in fn(dev)]


def test_config1_bias_relu_scale_rowsum_forward_backward(oracle, b200):
    """out = relu(A + b) * s; r = sum(out, dim=1); backward of sum(r): dA, db (sum over dim 0), ds."""
    m, n = 512, 768
    A0 = Tensor.randn_on([m, n], 1, Device(oracle, 0)).numpy()
    b0 = Tensor.randn_on([1, n], 2, Device(oracle, 0)).numpy()
    s0 = Tensor.randn_on([m, 1], 3, Device(oracle, 0)).numpy()

    def step(dev):
        A, b, s = (Tensor.from_numpy(v, dev, True) for v in (A0, b0, s0))
        out = (A + b).relu() * s
        r = out.sum_dim(1)
        total = out.sum()
        total.backward()
        return [out, r, total, A.grad, b.grad, s.grad]

    got, want = run_on(b200, step), run_on(oracle, step)
    for name, g, w in zip(["out", "r", "total", "dA", "db", "ds"], got, want):
        assert_bit_equal(f"config 1 {name}", g, w, zero_sign_matters=False)


def test_config3_mlp_elementwise_and_sgd(oracle, b200):
    """ReLU forward/backward on [32, W] activations, mse_loss mean, and the SGD update p -= 0.01*g."""
    W = 1024
    cpu = Device(oracle, 0)
    act0 = Tensor.randn_on([32, W], 5, cpu).numpy()
    tgt0 = Tensor.randn_on([32, W], 6, cpu).numpy()
    p0 = Tensor.randn_on([W, W], 11, cpu).numpy() * np.float32(0.02)
    g0 = Tensor.randn_on([W, W], 12, cpu).numpy() * np.float32(1e-3)

    def step(dev):
        a = Tensor.from_numpy(act0, dev, True)
        loss = mse_loss(a.relu(), Tensor.from_numpy(tgt0, dev))
        loss.backward()
        p = Tensor.from_numpy(p0, dev)
        p.grad = Tensor.from_numpy(g0, dev)
        SGD([p], 0.01).step()
        return [loss, a.grad, p]

    got, want = run_on(b200, step), run_on(oracle, step)
    for name, g, w in zip(["loss", "dact", "param"], got, want):
        assert_bit_equal(f"config 3 {name}", g, w, zero_sign_matters=False)


@pytest.mark.parametrize("transposed", [False, True])
def test_config4_softmax_from_primitives(oracle, b200, transposed):
    """Y = X + m1 + m2; M = max(Y, -1); E = exp(Y - M); S = sum(E, -1); P = E / S; X optionally a
    transposed (non-contiguous) view on its last two dims."""
    B, R, Cn = 4, 96, 128
    cpu = Device(oracle, 0)
    X0 = Tensor.randn_on([B, R, Cn], 21, cpu).numpy() * np.float32(2.0)
    m10 = Tensor.randn_on([B, 1, Cn], 22, cpu).numpy()
    m20 = synth.softmax_mask(R)

    def step(dev):
        m1, m2 = Tensor.from_numpy(m10, dev), Tensor.from_numpy(m20, dev)
        if transposed:
            # X is stored as [B, Cn, R]; the op reads it through strides (R*Cn, 1, R) as [B, R, Cn].
            from pytorches_b200.core import Operand, broadcast_strides, run_op
            Xs = Tensor.from_numpy(np.ascontiguousarray(X0.transpose(0, 2, 1)), dev)
            shape = [B, R, Cn]
            Y1 = run_op(dev, op.ADD, [0], [Operand(Xs, shape, [R * Cn, 1, R]), Operand(m1, shape, broadcast_strides(m1.shape, shape))], shape)
        else:
            Y1 = Tensor.from_numpy(X0, dev) + m1
        Y = Y1 + m2
        M = Y.max_dim(2, keepdim=True)
        E = (Y - M).exp()
        S = E.sum_dim(2, keepdim=True)
        return [Y, M, E, S, E / S]

    got, want = run_on(b200, step), run_on(oracle, step)
    for name, g, w in zip(["Y", "M", "E", "S", "P"], got, want):
        assert_bit_equal(f"config 4 {name}", g, w, zero_sign_matters=False)


def test_config2_full_reductions(oracle, b200):
    """sum, mean, max, argmax over a 2^22-element uniform[-1,1) tensor."""
    x0 = lcg_data(1 << 22, 7)

    def step(dev):
        x = Tensor.from_numpy(x0, dev)
        return [x.sum(), x.mean(), x.max(), x.argmax()]

    got, want = run_on(b200, step), run_on(oracle, step)
    for name, g, w in zip(["sum", "mean", "max"], got, want):
        assert_bit_equal(f"config 2 {name}", g, w)
    assert got[3] == want[3]
    ref = x0.astype(np.float64).sum()
    assert abs(float(got[0]) - ref) <= 1e-5 * 22 * np.abs(x0.astype(np.float64)).sum()


# ---- the same configurations at the benchmark's FULL sizes ----------------------------------------------
# The oracle finishes these in about a second each, so they are compared bit for bit as well.

def test_config1_full_size_bit_exact(oracle, b200):
    m = n = 4096
    cpu = Device(oracle, 0)
    A0, b0, s0 = (Tensor.randn_on(sh, seed, cpu).numpy() for sh, seed in (([m, n], 1), ([1, n], 2), ([m, 1], 3)))

    def step(dev):
        A, b, s = (Tensor.from_numpy(v, dev, True) for v in (A0, b0, s0))
        out = (A + b).relu() * s
        r = out.sum_dim(1)
        out.sum().backward()
        return [r, A.grad, b.grad, s.grad]

    got, want = run_on(b200, step), run_on(oracle, step)
    for name, g, w in zip(["r", "dA", "db", "ds"], got, want):
        assert_bit_equal(f"config 1 full size {name}", g, w, zero_sign_matters=False)


def test_config4_full_size_bit_exact(oracle, b200):
    if b200.device_info(0).free_memory < 24 * (1 << 30):
        pytest.skip("needs 24 GiB of free device memory")
    B, R, Cn = 64, 2048, 2048
    cpu = Device(oracle, 0)
    X0 = Tensor.randn_on([B, R, Cn], 21, cpu).numpy() * np.float32(2.0)
    m10 = Tensor.randn_on([B, 1, Cn], 22, cpu).numpy()
    m20 = synth.softmax_mask(R)

    def step(dev):
        Y = Tensor.from_numpy(X0, dev) + Tensor.from_numpy(m10, dev) + Tensor.from_numpy(m20, dev)
        M = Y.max_dim(2, keepdim=True)
        E = (Y - M).exp()
        del Y
        S = E.sum_dim(2, keepdim=True)
        P = E / S
        del E
        return [M, S, P]

    got = run_on(b200, step)
    want = run_on(oracle, step)
    for name, g, w in zip(["M", "S", "P"], got, want):
        assert_bit_equal(f"config 4 full size {name}", g, w)


def test_config2_full_size_against_oracle(oracle, b200):
    """The benchmark's own tensor, 2^28 elements uniform[-1, 1) from seed 7: sum and mean bit-equal to the
    oracle's, max and argmax exact."""
    x0 = synth.uniform_pm1(1 << 28, 7)

    def step(dev):
        x = Tensor.from_numpy(x0, dev)
        return [x.sum(), x.mean(), x.max(), x.argmax()]

    got, want = run_on(b200, step), run_on(oracle, step)
    for name, g, w in zip(["sum", "mean", "max"], got, want):
        assert_bit_equal(f"config 2 full size {name}", g, w)
    assert got[3] == want[3]

