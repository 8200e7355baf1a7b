"""Pins the CPU oracle to the reference's own test vectors (CPU run, no GPU needed).

Every check in ``conformance`` is a port of a reference test; running them against the oracle is what
makes the oracle trustworthy as the parity checker for the B200 plugin.
"""

import ctypes

import numpy as np
import pytest

import conformance
from harness import lcg_data


@pytest.mark.parametrize("check", conformance.ALL_CHECKS, ids=lambda f: f.__name__)
def test_oracle_passes_reference_case(oracle, check):
    check(oracle)


def test_oracle_takes_the_avx2_paths(oracle):
    """The bits of exp/log/tanh/axpy/sum depend on the AVX2+FMA code paths (plugins/cpu/src/simd.rs:6-15)."""
    fn = oracle.lib.cpuref_has_avx2
    fn.restype = ctypes.c_int
    assert fn() == 1, "this host lacks AVX2+FMA: oracle bits would follow the scalar paths"


def test_lcg_matches_scalar_definition():
    """harness.lcg_data against the scalar recurrence of plugins/cpu/tests/kernels.rs:13-21."""
    M = (1 << 64) - 1
    s = (5 * 6364136223846793005 + 1442695040888963407) & M
    want = []
    for _ in range(257):
        s = (s * 6364136223846793005 + 1442695040888963407) & M
        want.append(np.float32(np.float32(s >> 40) / np.float32(8388608.0)) - np.float32(1.0))
    assert np.array_equal(lcg_data(257, 5), np.array(want, dtype=np.float32))
