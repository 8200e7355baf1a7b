"""Recorded call lists replayed by the plugin (GPU run), and what the recorder writes down (CPU run).

``pytorches_b200_replay`` issues a host's recorded alloc / execute / free calls from native code. It
must compute what the same calls compute when the host issues them one by one: these tests run a step
through the Python mirror of the reference core with a recorder in between, replay the list several
times, and compare the results bit for bit with the step's own (and with the CPU oracle's).
"""

import ctypes

import numpy as np
import pytest

from harness import assert_bit_equal, lcg_data
from pytorches_b200 import abi
from pytorches_b200.abi import op
from pytorches_b200.core import Device, Tensor
from pytorches_b200.replay import CALL_ALLOC, CALL_EXECUTE, CALL_FREE, Recorder, algorithmic_bytes


def _step(dev, A0, b0, s0):
    A, b, s = (Tensor.from_numpy(v, dev, True) for v in (A0, b0, s0))
    out = (A + b).relu() * s
    r = out.sum_dim(1)
    out.sum().backward()
    return [r, A.grad, b.grad, s.grad]


def test_recorder_writes_down_every_call_in_order(oracle):
    """CPU run, against the oracle plugin: allocs get slots, frees name them, executes name slots for
    results made inside the step and raw pointers for tensors that existed before it."""
    rec = Recorder(oracle)
    dev = Device(rec, 0)
    x = Tensor.from_numpy(lcg_data(1000, 1), dev)
    rec.start()
    y = x.raw_unary(op.NEG)
    m = x.mean()
    del y
    step = rec.finish(0, keep=[x])
    kinds = [step.calls[i].kind for i in range(step.n)]
    # NEG: alloc + execute; mean: alloc sum, SUM_AXIS, alloc scalar, FILL, alloc quotient, DIV, free scalar, free sum; free y
    assert kinds.count(CALL_ALLOC) == 4 and kinds.count(CALL_EXECUTE) == 4 and kinds.count(CALL_FREE) == 3
    neg = step.calls[1]
    assert neg.kind == CALL_EXECUTE and neg.op == op.NEG and neg.ins[0].slot == -1 and neg.ins[0].data == x.buffer.ptr
    assert neg.outs[0].slot == 0 and neg.outs[0].ndim == 1 and neg.outs[0].shape[0] == 1000
    assert step.executes == 4 and step.peer_calls == 0
    # NEG 8n, SUM_AXIS 4n + 4, FILL 4, DIV 12
    assert algorithmic_bytes(step) == 8 * 1000 * 4 // 4 + 4 * 1000 + 4 + 4 + 12
    del m


@pytest.mark.gpu
def test_replayed_step_equals_the_step_itself(oracle, b200):
    m, n = 512, 768
    cpu = Device(oracle, 0)
    A0, b0, s0 = (Tensor.randn_on(sh, seed, cpu).numpy() for sh, seed in (([m, n], 1), ([1, n], 2), ([m, 1], 3)))
    want = [t.numpy() for t in _step(cpu, A0, b0, s0)]
    rec = Recorder(b200)
    dev = Device(rec, 0)
    A, b, s = (Tensor.from_numpy(v, dev, True) for v in (A0, b0, s0))
    # Results go into buffers that exist before the recording, so that they can be read after a replay.
    outs = [Tensor.zeros_on(sh, dev) for sh in ([m], [m, n], [1, n], [m, 1])]
    rec.start()
    for t in (A, b, s):
        t.grad = None
    out = (A + b).relu() * s
    r = out.sum_dim(1)
    out.sum().backward()
    for src, dst in zip((r, A.grad, b.grad, s.grad), outs):
        dev.plugin.execute(0, op.COPY, [0], [abi.Arg(src.buffer.ptr, tuple(src.shape), tuple(abi.contiguous_strides(src.shape)))],
                           [abi.Arg(dst.buffer.ptr, tuple(dst.shape), tuple(abi.contiguous_strides(dst.shape)))])
    del out, r
    for t in (A, b, s):
        t.grad = None
    step = rec.finish(0, keep=[A, b, s] + outs)
    for name, o, w in zip(["r", "dA", "db", "ds"], outs, want):
        assert_bit_equal(f"recorded step {name}", o.numpy(), w, zero_sign_matters=False)
    for o in outs:  # wipe, replay three times, compare again
        dev.plugin.execute(0, op.FILL, [0], [], [abi.Arg(o.buffer.ptr, tuple(o.shape), tuple(abi.contiguous_strides(o.shape)))])
    step.run(3)
    for name, o, w in zip(["r", "dA", "db", "ds"], outs, want):
        assert_bit_equal(f"replayed step {name}", o.numpy(), w, zero_sign_matters=False)


@pytest.mark.gpu
def test_back_to_back_reductions_keep_their_results_when_launches_overlap(b200):
    """Long full-tensor reductions issued back to back start while the one before is finishing. Every
    result must still be its own: sum, mean, max and argmax of different tensors, four steps per replay,
    against the same ops issued one by one with a synchronize after each."""
    rec = Recorder(b200)
    dev = Device(rec, 0)
    n = (1 << 24) + 65536 * 3
    xs = [Tensor.rand_uniform_on([n], 70 + k, -1.0, 1.0, dev) for k in range(4)]
    want = []
    for k, x in enumerate(xs):
        for fn in (x.sum, x.mean, x.max, x.argmax):
            want.append(fn().numpy())
            dev.synchronize()
    res = [Tensor(type(xs[0].buffer)(dev, 1, 8), [], dtype=abi.DTYPE_I64 if j % 4 == 3 else abi.DTYPE_F32) for j in range(16)]
    rec.start()
    j = 0
    for x in xs:
        flat = abi.Arg(x.buffer.ptr, (n,), (1,))
        for code, dt in ((op.SUM_AXIS, abi.DTYPE_F32), (None, abi.DTYPE_F32), (op.MAX_AXIS, abi.DTYPE_F32), (op.ARGMAX_AXIS, abi.DTYPE_I64)):
            if code is None:  # mean as the core issues it; its result is copied into the fixed buffer
                mval = x.mean()
                dev.plugin.execute(0, op.COPY, [0], [abi.Arg(mval.buffer.ptr, (), ())], [abi.Arg(res[j].buffer.ptr, (), ())])
                del mval
            else:
                dev.plugin.execute(0, code, [0], [flat], [abi.Arg(res[j].buffer.ptr, (), (), dt)])
            j += 1
    step = rec.finish(0, keep=xs + res)
    step.run(5)
    for j, (r, w) in enumerate(zip(res, want)):
        got = r.numpy()
        assert got.tobytes() == w.tobytes(), f"reduction {j}: {got} vs {w}"


@pytest.mark.gpu
def test_replay_reports_a_failing_call(b200):
    rec = Recorder(b200)
    dev = Device(rec, 0)
    x = Tensor.from_numpy(lcg_data(64, 1), dev)
    rec.start()
    y = x.raw_unary(op.NEG)
    step = rec.finish(0, keep=[x])
    step.calls[1].op = 9999  # not an op
    with pytest.raises(abi.PluginError) as err:
        step.run(2)
    assert err.value.status == abi.STATUS_UNSUPPORTED
    fn = b200.lib.pytorches_b200_replay
    assert fn(0, None, 3, 1, 0) == abi.STATUS_INVALID_ARGUMENT
    del y
