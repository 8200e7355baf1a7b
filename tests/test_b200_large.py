"""Sizes past 2^31 and 2^32 elements through size-independent properties (GPU run).

The oracle cannot chew through tens of GiB in seconds, so these check properties that pin every
element: an elementwise result whose max and min are both the one expected value has been written
correctly everywhere; a sum of ones has a known value under the reference's summation order; a planted
maximum must be found at its (large) position.
"""

import math

import numpy as np
import pytest

from pytorches_b200.abi import op
from pytorches_b200.core import Device, Operand, Tensor, run_op

pytestmark = pytest.mark.gpu


def _need(b200, gib):
    if b200.device_info(0).free_memory < gib * (1 << 30):
        pytest.skip(f"needs {gib} GiB of free device memory")


def test_two_to_the_31_elements_flat_ops_and_reductions(b200):
    """The largest contiguous size of the benchmark sweep: 2^31 elements (8 GiB per tensor), plus a ragged tail."""
    _need(b200, 40)
    dev = Device(b200, 0)
    n = (1 << 31) + 5
    a, b = Tensor.full_on([n], 1.0, dev), Tensor.full_on([n], 2.0, dev)
    out = a + b
    assert out.max().item() == 3.0 and (-out).max().item() == -3.0  # every element is exactly 3.0
    del out
    # Sum of n ones in the reference's order: 32768 full blocks of 65536 (exact), then 0.0 + ... in block
    # order stays exact up to 2^31, and the last block's 5.0 is absorbed by rounding (ulp is 256 there).
    assert a.sum().item() == float(1 << 31)
    a.axpy_(0.5, b)                                  # in place: 1 + 0.5*2 = 2
    assert a.max().item() == 2.0 and (-a).max().item() == -2.0
    e = b.raw_unary(op.EXP)
    assert abs(e.max().item() - math.exp(2.0)) < 1e-5 and abs((-e).max().item() + math.exp(2.0)) < 1e-5
    assert b.argmax().item() == 0                    # all equal: the first position


def test_more_than_two_to_the_32_elements_through_the_64_bit_row_kernel(b200):
    """[3, m] with odd m and 3m > 2^32: the broadcast row kernel runs with 64-bit work-item indices and
    scalar accesses; a column-vector addend plants the maximum in the last row."""
    _need(b200, 60)
    dev = Device(b200, 0)
    m = 1431655767
    assert m % 2 == 1 and 3 * m > (1 << 32)
    base = Tensor.full_on([3, m], 1.0, dev)
    c = Tensor.from_numpy(np.array([[0.0], [0.0], [4.0]], dtype=np.float32), dev)
    y = base + c
    del base
    flat = y.raw_reshape([3 * m])
    assert flat.max().item() == 5.0
    assert flat.argmax().item() == 2 * m             # first element of the last row, beyond 2^31
    rows = y.max_dim(1).numpy()
    assert rows.tolist() == [1.0, 1.0, 5.0]
    assert (-y).max_dim(1).numpy().tolist() == [-1.0, -1.0, -5.0]
