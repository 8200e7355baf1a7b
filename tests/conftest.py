import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

ORACLE_SO = os.path.join(ROOT, "oracle", "_build", "pytorches_plugin_cpuref.so")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def oracle():
    """The CPU oracle plugin (C++ restatement of the reference CPU plugin), built on demand."""
    from pytorches_b200.abi import Plugin

    if not os.path.exists(ORACLE_SO):
        subprocess.run(["make", "-C", os.path.join(ROOT, "oracle")], check=True, capture_output=True)
    return Plugin(ORACLE_SO)


@pytest.fixture(scope="session")
def b200():
    """The B200 plugin with at least one device; GPU tests only."""
    import pytorches_b200

    plugin = pytorches_b200.load_plugin()
    if plugin.device_count() == 0:
        pytest.fail("pytorches_plugin_b200.so reports no CUDA device on a GPU test run")
    return plugin
