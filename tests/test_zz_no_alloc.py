"""The allocation-free sum entry point against the vtable's SUM_AXIS (GPU run; collected last on purpose).

``pytorches_b200_sum_noalloc`` serves hosts that cannot allocate device memory at call time (their
GPU memory is already committed to a pool of their own, or allocator calls are banned from their hot
path because they can stall the device). It must give exactly what SUM_AXIS gives, call after call,
although all calls share one built-in scratch array that still holds the previous call's partial sums.
"""

import ctypes

import numpy as np
import pytest

from harness import Buf, assert_bit_equal, exec_op, lcg_data
from pytorches_b200 import abi
from pytorches_b200.abi import op

pytestmark = pytest.mark.gpu


def _entry(plugin):
    fn = plugin.lib.pytorches_b200_sum_noalloc
    fn.restype = ctypes.c_int32
    fn.argtypes = [ctypes.c_uint32, ctypes.c_void_p, ctypes.c_uint64, ctypes.c_void_p, ctypes.c_void_p]
    stream = plugin.lib.pytorches_b200_stream
    stream.restype, stream.argtypes = ctypes.c_void_p, [ctypes.c_uint32]
    return fn, stream(0)


def test_noalloc_sum_matches_sum_axis_on_consecutive_calls(b200):
    fn, stream = _entry(b200)
    # Two calls in a row that both go through the shared scratch (more than one 65536-block), the
    # second with fewer blocks than the first so stale partials sit right behind the ones it uses;
    # then the paths that bypass the scratch. Same tolerance as the SUM_AXIS parity tests: bit-exact.
    for n, seed in [(65536 * 37 + 1234, 21), (65536 * 5 + 77, 22), (65536 * 37 + 1234, 23), (40_000, 24), (17, 25), (0, 26)]:
        x = Buf(b200, lcg_data(n, seed))
        want = Buf.empty(b200, 1)
        assert exec_op(b200, op.SUM_AXIS, [0], [(x, (n,), (1,))], want, ()) == abi.STATUS_OK, b200.last_error()
        got = Buf.empty(b200, 1)
        assert fn(0, x.ptr, n, got.ptr, stream) == abi.STATUS_OK, b200.last_error()
        assert_bit_equal(f"noalloc sum n={n}", got.get(), want.get())


def test_noalloc_sum_on_the_default_stream_and_leaves_the_current_device_alone(b200):
    """``stream`` = NULL is CUDA's default stream. The call must not change the calling thread's
    current device (a host framework set it for its own work)."""
    import torch

    fn, _ = _entry(b200)
    n = 65536 * 11 + 321
    x = Buf(b200, lcg_data(n, 31))
    want = Buf.empty(b200, 1)
    assert exec_op(b200, op.SUM_AXIS, [0], [(x, (n,), (1,))], want, ()) == abi.STATUS_OK, b200.last_error()
    b200.synchronize(0)  # x is complete before a kernel on another stream reads it
    before = torch.cuda.current_device()
    got = Buf.empty(b200, 1)
    b200.synchronize(0)
    for _ in range(2):
        assert fn(0, x.ptr, n, got.ptr, None) == abi.STATUS_OK, b200.last_error()
    torch.cuda.synchronize()
    assert torch.cuda.current_device() == before
    assert_bit_equal("noalloc sum on the default stream", got.get(), want.get())


def test_noalloc_sum_rejects_sizes_beyond_its_scratch(b200):
    fn, stream = _entry(b200)
    x = Buf(b200, lcg_data(64, 1))
    out = Buf(b200, np.array([123.0], dtype=np.float32))
    assert fn(0, x.ptr, (1 << 32) + 1, out.ptr, stream) == abi.STATUS_INVALID_ARGUMENT
    assert "4294967296" in b200.last_error()
    b200.synchronize(0)
    assert out.get()[0] == 123.0  # nothing was launched
    assert fn(99, x.ptr, 64, out.ptr, stream) == abi.STATUS_INVALID_ARGUMENT
