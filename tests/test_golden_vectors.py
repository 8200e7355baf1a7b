"""Committed golden vectors (tests/golden/cpuref_vectors.npz, made by tests/golden/make_golden.py).

CPU run: the oracle still computes exactly what was frozen. GPU run: so does the B200 plugin.
"""

import importlib.util
import os

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
spec = importlib.util.spec_from_file_location("make_golden", os.path.join(HERE, "golden", "make_golden.py"))
make_golden = importlib.util.module_from_spec(spec)
spec.loader.exec_module(make_golden)
GOLDEN = np.load(os.path.join(HERE, "golden", "cpuref_vectors.npz"))


def _check(plugin):
    got = make_golden.run(plugin)
    assert sorted(got) == sorted(GOLDEN.files)
    for name in GOLDEN.files:
        g, w = got[name], GOLDEN[name]
        same = (g.view(np.uint32) == w.view(np.uint32)) | (np.isnan(g) & np.isnan(w)) | ((g == 0) & (w == 0) & (name == "relu"))
        assert same.all(), f"{name}: {np.flatnonzero(~same)[:5]} differ"


def test_oracle_matches_golden_vectors(oracle):
    _check(oracle)


@pytest.mark.gpu
def test_b200_matches_golden_vectors(b200):
    _check(b200)
