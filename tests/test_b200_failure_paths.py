"""Failure detection without faulting the GPU (GPU run).

Device-side waits in the staged kernels are bounded; an expired wait must surface as an error status
from the next blocking call and leave the device usable. The expiry is provoked by a self-test kernel
that waits, briefly, for bytes nobody sends. Host-side failures (bad arguments, absurd allocations)
are covered by ``conformance.check_errors_are_statuses``.
"""

import ctypes

import numpy as np
import pytest

from harness import Buf, assert_bit_equal, exec_op, lcg_data
from pytorches_b200 import abi
from pytorches_b200.abi import op

pytestmark = pytest.mark.gpu


def test_expired_device_wait_is_reported_once_and_device_stays_usable(b200):
    fn = b200.lib.pytorches_b200_selftest_expired_wait
    fn.restype, fn.argtypes = ctypes.c_int32, [ctypes.c_uint32, ctypes.c_void_p]
    stream = b200.lib.pytorches_b200_stream
    stream.restype, stream.argtypes = ctypes.c_void_p, [ctypes.c_uint32]
    b200.synchronize(0)  # clean slate
    assert fn(0, stream(0)) == abi.STATUS_OK
    with pytest.raises(abi.PluginError) as err:
        b200.synchronize(0)
    assert err.value.status == abi.STATUS_INTERNAL and "bounded" in str(err.value)
    b200.synchronize(0)  # reported once; the device is fine
    n = 65536 * 9 + 5    # and the kernels with bounded waits still give the right answer
    x = Buf(b200, lcg_data(n, 3))
    out = Buf.empty(b200, 1)
    assert exec_op(b200, op.SUM_AXIS, [0], [(x, (n,), (1,))], out, ()) == abi.STATUS_OK
    got = out.get()
    assert np.isfinite(got[0]) and abs(float(got[0]) - float(lcg_data(n, 3).astype(np.float64).sum())) < 1e-2 * n ** 0.5


def test_out_of_memory_is_a_status_and_the_cache_is_given_back(b200):
    """docs/plugin-abi.md:126-130: an allocation that cannot fit fails with OUT_OF_MEMORY, after the
    plugin has released its cache; everything keeps working afterwards."""
    total = b200.device_info(0).total_memory
    held = [b200.alloc(0, 256 << 20) for _ in range(4)]
    for h in held:
        b200.free(0, h)  # now cached inside the plugin
    with pytest.raises(abi.PluginOutOfMemory):
        b200.alloc(0, total + 1)
    big = b200.alloc(0, int(total * 0.6))  # needs the cached blocks to have been returnable
    b200.free(0, big)
    x = Buf(b200, lcg_data(100, 1))
    out = Buf.empty(b200, 100)
    assert exec_op(b200, op.NEG, [0], [(x, (100,), (1,))], out, (100,)) == abi.STATUS_OK
    assert_bit_equal("neg after OOM", out.get(), -lcg_data(100, 1))
