"""The reference's own test cases, run against the B200 plugin through the C ABI (GPU run)."""

import pytest

import conformance

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("check", conformance.ALL_CHECKS, ids=lambda f: f.__name__)
def test_b200_passes_reference_case(b200, check):
    check(b200)


def test_device_info(b200):
    from pytorches_b200 import abi

    info = b200.device_info(0)
    assert info.kind == abi.KIND_CUDA
    assert info.name and len(info.name) <= 63
    assert 0 < info.free_memory <= info.total_memory
    assert info.flags == 0


def test_work_runs_on_the_gpu(b200):
    """Every op is a kernel launch of this library: the launch counter moves."""
    import ctypes

    import numpy as np
    from harness import Buf, exec_op, lcg_data
    from pytorches_b200.abi import op

    fn = b200.lib.pytorches_b200_kernel_launches
    fn.restype = ctypes.c_uint64
    before = fn()
    x = Buf(b200, lcg_data(1000, 1))
    out = Buf.empty(b200, 1000)
    assert exec_op(b200, op.NEG, [0], [(x, (1000,), (1,))], out, (1000,)) == 0
    assert np.array_equal(out.get(), -lcg_data(1000, 1))
    assert fn() == before + 1
