"""Plugin-agnostic conformance checks, ported from the reference's own tests.

The reference describes, as intended future work, one harness that loads a plugin library and runs
the whole contract against it (docs/plugin-abi.md:255-262). This module is that harness for the ops
of this path: ``python -m pytorches_b200.conformance path/to/pytorches_plugin_X.so`` runs every check
against device 0 of any library that exports the ABI and exits non-zero if one fails.

Each ``check_*`` takes a loaded plugin and drives it through the vtable only. The same functions
run against the CPU oracle (CPU test run: this is how the oracle is pinned to the reference's
vectors) and against the B200 plugin (GPU test run). Two checks compare with PyTorch on the CPU and
are skipped by the command line tool when PyTorch is not installed. Sources:
  plugins/cpu/tests/kernels.rs          kernel cases, tolerances, determinism, allocator reuse
  crates/core/src/lib.rs:830-966        exact small autograd cases, RAND_NORMAL golden values, typed errors
  tests/diff/test_ops.py:31-57,107-138  forward + gradients against PyTorch CPU
"""

from __future__ import annotations

import math
import struct

import numpy as np

try:  # only the two *_against_torch checks need it
    import torch
except ImportError:  # pragma: no cover - the image used for development has it
    torch = None

from pytorches_b200 import abi
from pytorches_b200.harness import Buf, assert_bit_equal, close, exec_op, lcg_data
from pytorches_b200.abi import DTYPE_I64, contiguous_strides, op
from pytorches_b200.core import SGD, Device, Tensor, mse_loss


def f32_bits(v: float) -> int:
    return struct.unpack("<I", struct.pack("<f", v))[0]


# ---- plugins/cpu/tests/kernels.rs ---------------------------------------------------------------

def check_binary_broadcast_patterns(p):
    """kernels.rs:125-163."""
    cases = [
        ((37, 91), (91, 1)),       # full rows
        ((37, 91), (1, 0)),        # column broadcast: [m,1] over n
        ((37, 91), (0, 0)),        # scalar
        ((4, 5, 6), (30, 6, 1)),   # full 3-D
        ((300_000,), (1,)),        # large, parallel
    ]
    fns = {op.ADD: np.add, op.SUB: np.subtract, op.MUL: np.multiply, op.DIV: np.divide}
    for shape, sa in cases:
        n = int(np.prod(shape))
        av = lcg_data(max(n, 1) * 2, 5)
        bv = lcg_data(max(n, 1) * 2, 6) + np.float32(1.5)
        a, b = Buf(p, av), Buf(p, bv)
        a_log = np.lib.stride_tricks.as_strided(av, shape=shape, strides=tuple(4 * s for s in sa))
        b_log = bv[:n].reshape(shape)
        for code, fn in fns.items():
            out = Buf.empty(p, n)
            st = exec_op(p, code, [0], [(a, shape, sa), (b, shape, contiguous_strides(shape))], out, shape)
            assert st == abi.STATUS_OK, p.last_error()
            want = fn(a_log, b_log).astype(np.float32).reshape(-1)
            got = out.get()
            close(f"binary {code} {shape} strides {sa}", got, want, 1e-6)
            # one IEEE operation per element: numpy computes the same bits
            assert_bit_equal(f"binary {code} {shape} strides {sa}", got, want)


SUM_SHAPES = [(1000,), (33, 17), (5, 4, 3), (70_001,), (3, 200_000), (100_000, 3), (2, 600, 5), (4, 4096, 70), (1, 1), (64, 4096)]


def check_sum_axis_layouts(p):
    """kernels.rs:165-195: f64 reference at rtol 1e-4, and a second run must be bit-identical."""
    for shape in SUM_SHAPES:
        n = int(np.prod(shape))
        xv = lcg_data(n, 7)
        x = Buf(p, xv)
        for axis in range(len(shape)):
            want = xv.reshape(shape).astype(np.float64).sum(axis=axis).astype(np.float32).reshape(-1)
            oshape = tuple(s for i, s in enumerate(shape) if i != axis)
            out, out2 = Buf.empty(p, want.size), Buf.empty(p, want.size)
            ins = [(x, shape, contiguous_strides(shape))]
            assert exec_op(p, op.SUM_AXIS, [axis], ins, out, oshape) == abi.STATUS_OK, p.last_error()
            close(f"sum {shape} axis {axis}", out.get(), want, 1e-4)
            assert exec_op(p, op.SUM_AXIS, [axis], ins, out2, oshape) == abi.STATUS_OK
            assert_bit_equal(f"sum {shape} axis {axis} determinism", out.get(), out2.get())


def edge_values() -> np.ndarray:
    """kernels.rs:199-204."""
    vals = [0.0, -0.0, 1e-45, 1e-40, 1e-38, 1e-10, 0.1, 0.5, 1.0, 10.0, 88.0, 88.4, 88.5, 88.7, 89.0, 100.0, 1e30, math.inf,
            -1e-45, -1e-10, -0.5, -10.0, -87.0, -88.0, -100.0, -104.0, -1e30, -math.inf, math.nan]
    v = np.array(vals, dtype=np.float32)
    a = np.arange(-300, 300, dtype=np.float32) * np.float32(0.37)
    b = np.arange(1, 2000, dtype=np.float32) * np.float32(1e-3)
    return np.concatenate([v, a, b])


def check_vector_math_edge_values(p):
    """kernels.rs:197-228: a few ulps against f64 truth, exact infinities and NaNs."""
    vals = edge_values()
    n = vals.size
    x = Buf(p, vals)
    f32max = float(np.finfo(np.float32).max)
    tiny = float(np.finfo(np.float32).tiny)
    for code, name, fn in [(op.EXP, "exp", np.exp), (op.LOG, "log", np.log), (op.TANH, "tanh", np.tanh)]:
        out = Buf.empty(p, n)
        assert exec_op(p, code, [0], [(x, (n,), (1,))], out, (n,)) == abi.STATUS_OK, p.last_error()
        got = out.get()
        with np.errstate(all="ignore"):
            want64 = fn(vals.astype(np.float64))
        for i in range(n):
            g, w, v = float(got[i]), float(want64[i]), float(vals[i])
            if math.isnan(w):
                assert math.isnan(g), f"{name}({v}) = {g}, want NaN (index {i})"
            elif math.isinf(w) or w > f32max:
                assert g == (math.inf if w > 0 else -math.inf), f"{name}({v}) = {g} (index {i})"
            else:
                w32 = float(np.float32(w))
                tol = 4e-7 * abs(w32) + 2e-45 + (tiny * 1e-1 if abs(w32) < tiny else 0.0)
                assert abs(g - w32) <= tol, f"{name}({v}) = {g}, want {w32} (index {i})"


def check_axpy(p):
    """kernels.rs:230-245."""
    alpha = f32_bits(-0.25)
    for n in [1, 7, 8, 33, 4097, 300_000]:
        av, bv = lcg_data(n, 8), lcg_data(n, 9)
        want = (av - np.float32(0.25) * bv).astype(np.float32)
        a, b = Buf(p, av), Buf(p, bv)
        sh, st = (n,), (1,)
        assert exec_op(p, op.AXPY, [alpha], [(a, sh, st), (b, sh, st)], a, sh) == abi.STATUS_OK, p.last_error()
        close(f"axpy in place n={n}", a.get(), want, 1e-6)
        a2, out = Buf(p, av), Buf.empty(p, n)
        assert exec_op(p, op.AXPY, [alpha], [(a2, sh, st), (b, sh, st)], out, sh) == abi.STATUS_OK
        close(f"axpy out of place n={n}", out.get(), want, 1e-6)


def check_transpose_and_strided_unary(p):
    """kernels.rs:247-268: exact."""
    for r, c in [(1, 9), (9, 1), (3, 5), (32, 32), (33, 31), (257, 129), (1000, 70)]:
        xv = lcg_data(r * c, 10)
        want = np.ascontiguousarray(xv.reshape(r, c).T).reshape(-1)
        x = Buf(p, xv)
        sh, st = (c, r), (1, c)
        out = Buf.empty(p, r * c)
        assert exec_op(p, op.COPY, [0], [(x, sh, st)], out, sh) == abi.STATUS_OK, p.last_error()
        assert_bit_equal(f"transpose {r}x{c}", out.get(), want)
        out = Buf.empty(p, r * c)
        assert exec_op(p, op.NEG, [0], [(x, sh, st)], out, sh) == abi.STATUS_OK
        assert_bit_equal(f"neg of transpose {r}x{c}", out.get(), -want)


def check_freed_buffers_are_reused(p):
    """kernels.rs:270-280."""
    a = p.alloc(0, 3 << 20)
    p.free(0, a)
    b = p.alloc(0, 3 << 20)
    assert a == b, "same-size allocation did not reuse the freed buffer"
    p.free(0, b)


def check_matmul(p):
    """kernels.rs:76-123: all transpose flag combinations, odd shapes, strided A; rtol 2e-6 vs f64."""
    for (m, k, n) in [(1, 1, 1), (5, 7, 3), (6, 16, 16), (7, 17, 33), (97, 255, 130), (100, 513, 200), (1, 300, 200), (300, 300, 1), (130, 1, 70), (250, 600, 250)]:
        av, bv = lcg_data(m * k, 1), lcg_data(k * n, 2)
        a, b = Buf(p, av), Buf(p, bv)
        for flags in range(4):
            if flags and not p.supports_op(op.MATMUL_T):
                continue
            ta, tb = bool(flags & 1), bool(flags & 2)
            sa = (k, m) if ta else (m, k)
            sb = (n, k) if tb else (k, n)
            A = av.reshape(sa).astype(np.float64)
            B = bv.reshape(sb).astype(np.float64)
            want = ((A.T if ta else A) @ (B.T if tb else B)).astype(np.float32).reshape(-1)
            out = Buf.empty(p, m * n)
            code = op.MATMUL if flags == 0 else op.MATMUL_T
            st = exec_op(p, code, [flags], [(a, sa, contiguous_strides(sa)), (b, sb, contiguous_strides(sb))], out, (m, n))
            assert st == abi.STATUS_OK, p.last_error()
            close(f"matmul {m}x{k}x{n} flags {flags}", out.get(), want, 2e-6)
    m, k, n = 13, 21, 17  # A is a transposed view of a [k, m] matrix passed through MATMUL strides
    av, bv = lcg_data(k * m, 3), lcg_data(k * n, 4)
    want = (av.reshape(k, m).T.astype(np.float64) @ bv.reshape(k, n).astype(np.float64)).astype(np.float32).reshape(-1)
    a, b, out = Buf(p, av), Buf(p, bv), Buf.empty(p, m * n)
    assert exec_op(p, op.MATMUL, [0], [(a, (m, k), (1, m)), (b, (k, n), (n, 1))], out, (m, n)) == abi.STATUS_OK
    close("strided matmul", out.get(), want, 2e-6)


# ---- crates/core/src/lib.rs tests, through the mini-core -----------------------------------------

RANDN_GOLDEN = [0.6574781, -0.08203645, -2.2065563, 0.70945626]  # crates/core/src/lib.rs:929-937


def check_randn(p):
    dev = Device(p, 0)
    v = Tensor.randn_on([4], 1234, dev).numpy()
    assert np.all(np.abs(v - np.array(RANDN_GOLDEN, dtype=np.float32)) < 1e-5), v
    a = Tensor.randn_on([100_000], 42, dev).numpy()  # lib.rs:913-926
    assert np.array_equal(a, Tensor.randn_on([100_000], 42, dev).numpy())
    assert not np.array_equal(a, Tensor.randn_on([100_000], 43, dev).numpy())
    assert abs(float(a.mean())) < 0.02 and abs(float(a.var()) - 1.0) < 0.03
    assert np.isfinite(a).all()


def check_core_exact_cases(p):
    dev = Device(p, 0)
    leaf = lambda data, shape: Tensor.from_numpy(np.array(data, dtype=np.float32).reshape(shape), dev, True)
    x = leaf([1, 2, 3], [3])  # square_grad, lib.rs:830-834
    (x * x).sum().backward()
    assert x.grad.numpy().tolist() == [2.0, 4.0, 6.0]
    x, b = leaf([1, 2, 3, 4, 5, 6], [2, 3]), leaf([10, 20, 30], [3])  # lib.rs:837-851
    assert (x + b).numpy().reshape(-1).tolist() == [11.0, 22.0, 33.0, 14.0, 25.0, 36.0]
    (x + b).sum().backward()
    assert x.grad.numpy().reshape(-1).tolist() == [1.0] * 6
    assert b.grad.numpy().tolist() == [2.0, 2.0, 2.0]
    a = Tensor.from_numpy(np.array([1, 2, 3], dtype=np.float32), dev)  # lib.rs:866-873
    a.axpy_(-0.5, Tensor.from_numpy(np.array([10, 20, 30], dtype=np.float32), dev))
    assert a.numpy().tolist() == [-4.0, -8.0, -12.0]
    x = leaf([1, 2, 3, 4, 5, 6], [2, 3])  # transpose_values, lib.rs:882-885
    assert x.t().numpy().reshape(-1).tolist() == [1.0, 4.0, 2.0, 5.0, 3.0, 6.0]
    x = leaf([3.0], [1])  # grads_accumulate_through_reuse, lib.rs:888-893
    ((x * x) + x).sum().backward()
    assert x.grad.numpy().tolist() == [7.0]
    t = Tensor.full_on([2, 2], 7.0, dev)  # fill, lib.rs:903-911
    assert t.numpy().reshape(-1).tolist() == [7.0] * 4
    assert Tensor.zeros_on([3], dev).numpy().tolist() == [0.0] * 3
    o = leaf([1.0, 2.0], [2])  # accumulate over two backward passes, test_ops.py:118-122
    (o * o).sum().backward()
    (o * o).sum().backward()
    assert o.grad.numpy().tolist() == [4.0, 8.0]


def check_errors_are_statuses(p):
    """lib.rs:948-966 and plugins/cpu/src/lib.rs:250-330: bad calls return statuses; the plugin stays usable."""
    x = Buf(p, lcg_data(12, 1))
    out = Buf.empty(p, 12)
    sh, st = (3, 4), (4, 1)
    ok = [(x, sh, st)]
    assert exec_op(p, 9999, [0], ok, out, sh) == abi.STATUS_UNSUPPORTED
    assert exec_op(p, op.NEG, [0], [], out, sh) == abi.STATUS_INVALID_ARGUMENT            # arity
    assert exec_op(p, op.ADD, [0], ok, out, sh) == abi.STATUS_INVALID_ARGUMENT             # arity
    assert exec_op(p, op.NEG, [0], [(x, (2, 4), (4, 1))], out, sh) == abi.STATUS_INVALID_ARGUMENT  # numel
    assert exec_op(p, op.ADD, [0], [(x, sh, st), (x, (4, 3), (3, 1))], out, sh) == abi.STATUS_INVALID_ARGUMENT
    assert exec_op(p, op.SUM_AXIS, [2], ok, out, (3,)) == abi.STATUS_INVALID_ARGUMENT      # axis out of range
    assert exec_op(p, op.SUM_AXIS, [-1], ok, out, (3,)) == abi.STATUS_INVALID_ARGUMENT
    assert exec_op(p, op.SUM_AXIS, [1], ok, out, (4,)) == abi.STATUS_INVALID_ARGUMENT      # wrong output size
    # two outputs
    o = abi.Arg(out.ptr, sh, st)
    assert p.execute_status(0, op.NEG, [0], [abi.Arg(x.ptr, sh, st)], [o, o]) == abi.STATUS_INVALID_ARGUMENT
    # a dtype the ABI does not have
    assert p.execute_status(0, op.NEG, [0], [abi.Arg(x.ptr, sh, st, 7)], [o]) == abi.STATUS_UNSUPPORTED
    assert p.last_error()
    # absurd allocation -> OUT_OF_MEMORY, quickly, and the plugin still works
    try:
        p.alloc(0, 1 << 60)
        raise AssertionError("alloc of 2^60 bytes succeeded")
    except abi.PluginOutOfMemory as e:
        assert "alloc" in str(e)
    assert exec_op(p, op.NEG, [0], ok, out, sh) == abi.STATUS_OK
    assert_bit_equal("neg after errors", out.get(), -lcg_data(12, 1))


def check_zero_sized_and_scalars(p):
    """docs/plugin-abi.md:170: ndim 0 and zero-element tensors are accepted."""
    dev = Device(p, 0)
    s = Tensor.scalar_on(2.5, dev)
    assert (s * s).numpy().item() == 6.25 and (s * s).shape == []
    e = Buf(p, np.zeros(0, dtype=np.float32))
    out = Buf.empty(p, 0)
    for code, ins, osh in [(op.NEG, [(e, (0,), (1,))], (0,)), (op.ADD, [(e, (0, 3), (3, 1)), (e, (0, 3), (3, 1))], (0, 3)),
                           (op.FILL, [], (0,)), (op.SUM_AXIS, [(e, (0, 3), (3, 1))], (0,)), (op.COPY, [(e, (4, 0), (0, 1))], (4, 0))]:
        assert exec_op(p, code, [1 if code == op.SUM_AXIS else 0], ins, out, osh) == abi.STATUS_OK, (code, p.last_error())
    z = Buf.empty(p, 3)  # summing a zero-length axis gives zeros (reduce.rs:106-109)
    assert exec_op(p, op.SUM_AXIS, [0], [(e, (0, 3), (3, 1))], z, (3,)) == abi.STATUS_OK
    assert z.get().tolist() == [0.0, 0.0, 0.0]


# ---- tests/diff/test_ops.py: forward and gradients against PyTorch CPU ---------------------------------

def _cases():
    randn = lambda *s: (lambda: torch.randn(*s))
    pos = lambda *s: (lambda: torch.rand(*s) + 0.5)
    return [
        ("add", lambda a, b: a + b, [randn(3, 4), randn(3, 4)]),
        ("add_broadcast_row", lambda a, b: a + b, [randn(3, 4), randn(4)]),
        ("add_broadcast_col", lambda a, b: a + b, [randn(3, 1), randn(1, 4)]),
        ("add_3d", lambda a, b: a + b, [randn(2, 3, 5), randn(3, 1)]),
        ("sub", lambda a, b: a - b, [randn(3, 4), randn(3, 4)]),
        ("sub_broadcast", lambda a, b: a - b, [randn(2, 3, 4), randn(3, 1)]),
        ("mul", lambda a, b: a * b, [randn(3, 4), randn(3, 4)]),
        ("mul_broadcast", lambda a, b: a * b, [randn(2, 3), randn(3)]),
        ("div", lambda a, b: a / b, [randn(3, 4), pos(3, 4)]),
        ("div_broadcast", lambda a, b: a / b, [randn(3, 4), pos(4)]),
        ("neg", lambda a: -a, [randn(5)]),
        ("exp", lambda a: a.exp(), [randn(3, 4)]),
        ("log", lambda a: a.log(), [pos(3, 4)]),
        ("relu", lambda a: a.relu(), [randn(4, 5)]),
        ("tanh", lambda a: a.tanh(), [randn(4, 5)]),
        ("transpose", lambda a: a.t(), [randn(3, 4)]),
        ("reshape", lambda a: a.reshape([4, 3]), [randn(2, 6)]),
        ("scalar_rsub", lambda a: 2.0 - a, [randn(3)]),
        ("scalar_rdiv", lambda a: 2.0 / a, [pos(3)]),
        ("reuse", lambda a: a * a + a, [randn(6)]),
        ("bias_relu_scale", lambda x, b, s: (x + b).relu() * s, [randn(8, 16), randn(1, 16), randn(8, 1)]),
    ]


def check_diff_against_torch(p, rtol=1e-5):
    """test_ops.py:66-105: atol = rtol * max(|want|, 1). The matmul cases are left to check_matmul."""
    torch.manual_seed(0)
    dev = Device(p, 0)

    def assert_close(got, want, what):
        got, want = torch.from_numpy(np.asarray(got, dtype=np.float32)), want.detach().to(torch.float32)
        assert list(got.shape) == list(want.shape), f"{what}: shape {list(got.shape)} vs {list(want.shape)}"
        scale = max(want.abs().max().item(), 1.0) if want.numel() else 1.0
        assert torch.allclose(got, want, rtol=rtol, atol=rtol * scale), f"{what}: max abs diff {(got - want).abs().max().item()}"

    for name, fn, gens in _cases():
        ref_in = [g().requires_grad_(True) for g in gens]
        ours_in = [Tensor.from_numpy(t.detach().numpy(), dev, True) for t in ref_in]
        ref_out, ours_out = fn(*ref_in), fn(*ours_in)
        assert_close(ours_out.numpy(), ref_out, f"{name} forward")
        (ref_out * ref_out).sum().backward()
        (ours_out * ours_out).sum().backward()
        for i, (r, o) in enumerate(zip(ref_in, ours_in)):
            assert o.grad is not None, f"{name}: input {i} has no grad"
            assert_close(o.grad.numpy(), r.grad, f"{name} grad[{i}]")
    for reduce in ("sum", "mean"):  # test_ops.py:107-115
        r = torch.randn(3, 4).requires_grad_(True)
        o = Tensor.from_numpy(r.detach().numpy(), dev, True)
        ro, oo = getattr(r, reduce)(), getattr(o, reduce)()
        assert abs(oo.item() - ro.item()) < 5e-4
        ro.backward()
        oo.backward()
        assert_close(o.grad.numpy(), r.grad, f"{reduce} grad")
    # an SGD step on an mse loss (crates/python/python/pytorches/nn.py:276-278, optim.py:13-16)
    w0, x0, t0 = torch.randn(5, 7), torch.randn(5, 7), torch.randn(5, 7)
    w = w0.clone().requires_grad_(True)
    torch.nn.functional.mse_loss(w * x0, t0).backward()
    w_ref = w.detach() - 0.1 * w.grad
    wo = Tensor.from_numpy(w0.numpy(), dev, True)
    mse_loss(wo * Tensor.from_numpy(x0.numpy(), dev), Tensor.from_numpy(t0.numpy(), dev)).backward()
    SGD([wo], 0.1).step()
    assert_close(wo.numpy(), w_ref, "sgd step")


# ---- appended ops: pinned to torch CPU (no reference implementation exists) ---------------------------

def check_max_argmax_against_torch(p):
    """MAX_AXIS / ARGMAX_AXIS (appended codes 203/204, optional): torch CPU's amax/argmax semantics."""
    if not (p.supports_op(op.MAX_AXIS) and p.supports_op(op.ARGMAX_AXIS)):
        return  # a plugin of the unextended ABI conforms without them
    rng = np.random.default_rng(3)
    shapes = [(1000,), (33, 17), (5, 4, 3), (70_001,), (3, 200_000), (100_000, 3), (2, 600, 5), (1, 1), (64, 4096), (7, 1, 9)]
    for shape in shapes:
        n = int(np.prod(shape))
        xv = lcg_data(n, 11)
        # ties: quantise so values repeat; NaNs: a few, to check they win
        xq = (np.round(xv * 8) / 8).astype(np.float32)
        xn = xv.copy()
        xn[rng.integers(0, n, size=max(1, n // 500))] = np.nan
        for tag, data in [("plain", xv), ("ties", xq), ("nan", xn)]:
            x = Buf(p, data)
            tx = torch.from_numpy(data.reshape(shape))
            for axis in range(len(shape)):
                oshape = tuple(s for i, s in enumerate(shape) if i != axis)
                m = int(np.prod(oshape)) if oshape else 1
                ins = [(x, shape, contiguous_strides(shape))]
                out = Buf.empty(p, m)
                assert exec_op(p, op.MAX_AXIS, [axis], ins, out, oshape) == abi.STATUS_OK, p.last_error()
                assert_bit_equal(f"max {tag} {shape} axis {axis}", out.get(), torch.amax(tx, dim=axis).numpy().reshape(-1), zero_sign_matters=False)
                iout = Buf.empty(p, m, dtype=np.int64)
                assert exec_op(p, op.ARGMAX_AXIS, [axis], ins, iout, oshape, DTYPE_I64) == abi.STATUS_OK, p.last_error()
                want = torch.argmax(tx, dim=axis).numpy().reshape(-1)
                got = iout.get()
                assert np.array_equal(got, want), f"argmax {tag} {shape} axis {axis}: first diff at {np.flatnonzero(got != want)[:3]}"
    # a zero-length reduced axis has no maximum
    e = Buf(p, np.zeros(0, dtype=np.float32))
    out = Buf.empty(p, 3)
    assert exec_op(p, op.MAX_AXIS, [0], [(e, (0, 3), (3, 1))], out, (3,)) == abi.STATUS_INVALID_ARGUMENT
    # f32 output descriptor for argmax is rejected: the op writes i64
    x = Buf(p, lcg_data(12, 1))
    assert exec_op(p, op.ARGMAX_AXIS, [0], [(x, (12,), (1,))], out, ()) == abi.STATUS_UNSUPPORTED  # also when the op is not offered at all


FUSED = {  # fused code -> (first op, second op, which input the first op reads: None = both)
    op.RELU_GRAD: (op.STEP, op.MUL),
    op.ADD_RELU: (op.ADD, op.RELU),
    op.SUB_EXP: (op.SUB, op.EXP),
}


def check_fused_ops_equal_their_sequences(p):
    """The appended optional ops 501-503 are defined as two reference ops run one after the other
    (docs/plugin-abi.md:285-287 names them as candidates; crates/core/src/lib.rs:639-643 is the relu
    gradient). A plugin need not offer them; one that does must give the sequence's bits on every layout."""
    offered = [c for c in FUSED if p.supports_op(c)]
    cases = [
        ((1000,), (1,), (1,)), ((4099,), (1,), (0,)), ((7,), (1,), (1,)), ((70_003,), (1,), (1,)),
        ((37, 91), (91, 1), (0, 1)), ((64, 128), (128, 1), (1, 0)), ((8, 16, 32), (512, 32, 1), (0, 1, 0)),
        ((33, 65), (1, 33), (65, 1)), ((8, 64, 128), (8192, 1, 64), (128, 0, 1)), ((2, 3, 4), (1, 2, 6), (12, 4, 1)), ((), (), ()),
    ]
    specials = np.array([0.0, -0.0, np.inf, -np.inf, np.nan, -3.0, 3.0, 1e-45, 89.0, -104.0], dtype=np.float32)
    for shape, sa, sb in cases:
        n = int(np.prod(shape)) if shape else 1
        span = lambda st: 1 + sum((d - 1) * t for d, t in zip(shape, st))
        av, bv = lcg_data(span(sa), 41) * np.float32(12.0), lcg_data(span(sb), 42)
        av[: min(av.size, specials.size)] = specials[: av.size]
        bv[: min(bv.size, specials.size)] = specials[::-1][: bv.size]
        a, b = Buf(p, av), Buf(p, bv)
        dense = tuple(contiguous_strides(shape))
        for code in offered:
            first, second = FUSED[code]
            fused, mid, seq = Buf.empty(p, n), Buf.empty(p, n), Buf.empty(p, n)
            assert exec_op(p, code, [0], [(a, shape, sa), (b, shape, sb)], fused, shape) == abi.STATUS_OK, p.last_error()
            if code == op.RELU_GRAD:  # MUL(g, STEP(x))
                assert exec_op(p, op.STEP, [0], [(b, shape, sb)], mid, shape) == abi.STATUS_OK
                assert exec_op(p, op.MUL, [0], [(a, shape, sa), (mid, shape, dense)], seq, shape) == abi.STATUS_OK
            else:
                assert exec_op(p, first, [0], [(a, shape, sa), (b, shape, sb)], mid, shape) == abi.STATUS_OK
                assert exec_op(p, second, [0], [(mid, shape, dense)], seq, shape) == abi.STATUS_OK
            assert_bit_equal(f"fused op {code} vs its sequence, {shape} {sa} {sb}", fused.get(), seq.get())
    # same arity and shape rules as the binary ops
    x = Buf(p, lcg_data(12, 1))
    out = Buf.empty(p, 12)
    for code in offered:
        assert exec_op(p, code, [0], [(x, (3, 4), (4, 1))], out, (3, 4)) == abi.STATUS_INVALID_ARGUMENT
        assert exec_op(p, code, [0], [(x, (3, 4), (4, 1)), (x, (4, 3), (3, 1))], out, (3, 4)) == abi.STATUS_INVALID_ARGUMENT
    # the host uses them only when offered, and gets the same values and gradients either way
    grads = {}
    for fused in (True, False):
        dev = Device(p, 0, fused=fused)
        A = Tensor.from_numpy(lcg_data(6 * 50, 7).reshape(6, 50), dev, requires_grad=True)
        bias = Tensor.from_numpy(lcg_data(50, 8).reshape(1, 50), dev, requires_grad=True)
        m = Tensor.from_numpy(lcg_data(6, 9).reshape(6, 1), dev, requires_grad=True)
        y = A.add_relu(bias).sub_exp(m).mul(A.relu())
        loss = y.sum()
        loss.backward()
        grads[fused] = [loss.numpy(), A.grad.numpy(), bias.grad.numpy(), m.grad.numpy()]
    for got, want in zip(grads[True], grads[False]):
        assert_bit_equal("fused vs unfused host sequences", got.reshape(-1), want.reshape(-1))


def check_concurrent_threads(p):
    """docs/plugin-abi.md:228-236: every entry point may be called from any number of threads; calls into
    one device behave as if serialized; last_error is per thread. Eight threads each run their own chain
    of allocations, ops, reductions and frees on device 0 at once; every result must be what the chain
    yields alone (the ops used are bit-exact), and a thread that provokes errors is the only one to see them."""
    import threading

    n_threads, rounds = 8, 12
    failures: list = []
    sums: dict = {}

    def size(tid, k):  # odd sizes, different per thread: different buckets and kernels; the last two
        return (1000 + 4099 * tid if tid < 6 else 66000 + 1111 * tid) + 37 * k  # reach the long-row reductions

    def sum_of(buf, n):
        r = Buf.empty(p, 1)
        assert exec_op(p, op.SUM_AXIS, [0], [(buf, (n,), (1,))], r, ()) == abi.STATUS_OK
        v = r.get()[0]
        r.free()
        return v
    start = threading.Barrier(n_threads)

    def expected(a, b, k):
        y = (a + b) * np.float32(k + 1)
        y = np.maximum(y, np.float32(0)) - a
        return y

    def worker(tid: int):
        try:
            start.wait()
            for k in range(rounds):
                n = size(tid, k)
                a_h, b_h = lcg_data(n, 100 + tid), lcg_data(n, 200 + tid + k)
                a, b = Buf(p, a_h), Buf(p, b_h)
                s = Buf(p, np.full(1, k + 1, dtype=np.float32))
                t0, t1, t2, out = (Buf.empty(p, n) for _ in range(4))
                sh, st = (n,), (1,)
                assert exec_op(p, op.ADD, [0], [(a, sh, st), (b, sh, st)], t0, sh) == abi.STATUS_OK
                assert exec_op(p, op.MUL, [0], [(t0, sh, st), (s, sh, (0,))], t1, sh) == abi.STATUS_OK
                assert exec_op(p, op.RELU, [0], [(t1, sh, st)], t2, sh) == abi.STATUS_OK
                assert exec_op(p, op.SUB, [0], [(t2, sh, st), (a, sh, st)], out, sh) == abi.STATUS_OK
                want = expected(a_h, b_h, k)
                assert_bit_equal(f"thread {tid} round {k}", out.get(), want)
                # a reduction too: it takes scratch from the allocator the other threads are using
                m = Buf.empty(p, 1)
                assert exec_op(p, op.MAX_AXIS, [0], [(out, sh, st)], m, ()) == abi.STATUS_OK
                assert m.get()[0] == want.max()
                sums[(tid, k)] = sum_of(out, n)
                if tid == 0:
                    # errors stay with the thread that made them
                    assert exec_op(p, 9999, [0], [(a, sh, st)], out, sh) == abi.STATUS_UNSUPPORTED
                    assert p.last_error()
                for buf in (a, b, s, t0, t1, t2, out, m):
                    buf.free()
        except BaseException as e:  # noqa: BLE001 - reported to the main thread
            failures.append((tid, repr(e)))
            try:
                start.abort()
            except Exception:
                pass

    threads = [threading.Thread(target=worker, args=(i,)) for i in range(n_threads)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not failures, failures
    # the ordered sums computed under contention carry the bits the same call yields alone
    for (tid, k), got in sorted(sums.items()):
        want = Buf(p, expected(lcg_data(size(tid, k), 100 + tid), lcg_data(size(tid, k), 200 + tid + k), k))
        alone = sum_of(want, size(tid, k))
        assert f32_bits(got) == f32_bits(alone), (tid, k, got, alone)
        want.free()
    # the main thread made no failing call since its last successful one: the others' errors are not its own
    x = Buf(p, lcg_data(8, 3))
    out = Buf.empty(p, 8)
    assert exec_op(p, op.NEG, [0], [(x, (8,), (1,))], out, (8,)) == abi.STATUS_OK
    assert_bit_equal("neg after threads", out.get(), -lcg_data(8, 3))


ALL_CHECKS = [
    check_binary_broadcast_patterns,
    check_sum_axis_layouts,
    check_vector_math_edge_values,
    check_axpy,
    check_transpose_and_strided_unary,
    check_freed_buffers_are_reused,
    check_matmul,
    check_randn,
    check_core_exact_cases,
    check_errors_are_statuses,
    check_zero_sized_and_scalars,
    check_diff_against_torch,
    check_max_argmax_against_torch,
    check_fused_ops_equal_their_sequences,
    check_concurrent_threads,
]


def main(argv=None) -> int:
    import argparse
    import sys
    import time
    import traceback

    ap = argparse.ArgumentParser(description="Run the plugin conformance checks against one plugin library.")
    ap.add_argument("library", help="path of a pytorches_plugin_*.so")
    ap.add_argument("-k", default="", help="only checks whose name contains this text")
    args = ap.parse_args(argv)
    plugin = abi.Plugin(args.library)  # applies the loader's vtable checks
    print(f"{plugin.name}: ABI {plugin.vt.abi_version}, {plugin.device_count()} device(s)")
    if plugin.device_count() == 0:
        print("no devices: nothing to check (a plugin without hardware must report zero devices quietly)")
        return 0
    failed = 0
    for check in ALL_CHECKS:
        if args.k not in check.__name__:
            continue
        if torch is None and check.__name__.endswith("_against_torch"):
            print(f"SKIP  {check.__name__} (PyTorch is not installed)")
            continue
        t = time.perf_counter()
        try:
            check(plugin)
            print(f"PASS  {check.__name__}  ({time.perf_counter() - t:.1f} s)")
        except Exception:  # noqa: BLE001 - report and go on to the next check
            failed += 1
            print(f"FAIL  {check.__name__}")
            traceback.print_exc(file=sys.stdout)
    print(f"{failed} check(s) failed" if failed else "all checks passed")
    return 1 if failed else 0


if __name__ == "__main__":
    raise SystemExit(main())
