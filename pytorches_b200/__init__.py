"""B200-native backend plugin for the pytorches tensor library's data-parallel hot path.

The product is the shared library ``pytorches_plugin_b200.so`` (built from ``csrc/``), which
implements the reference's plugin C ABI with hand-written sm_100a kernels. The Python modules are
the host side a maintainer of the reference would recognise: ``abi`` binds any plugin through the
C ABI, ``core`` replays the reference core's op sequences, ``shard`` splits them across GPUs.
"""

import os

from . import abi
from .abi import Plugin

__all__ = ["abi", "Plugin", "plugin_path", "load_plugin"]

PLUGIN_FILE = "pytorches_plugin_b200.so"


def plugin_path() -> str:
    """Where the built plugin lives: next to its sources, under ``csrc/``."""
    return os.path.join(os.path.dirname(os.path.abspath(__file__)), "csrc", PLUGIN_FILE)


_PLUGIN = None


def load_plugin() -> Plugin:
    """Load the B200 plugin (once per process). Fails loudly when it has not been built."""
    global _PLUGIN
    if _PLUGIN is None:
        override = os.environ.get("PYTORCHES_B200_PLUGIN")  # a library built elsewhere (no check against the sources beside this package)
        if override:
            _PLUGIN = Plugin(override)
            return _PLUGIN
        path = plugin_path()
        if not os.path.exists(path):
            raise RuntimeError(
                f"{path} is missing: build it with `python -m pytorches_b200.build` "
                "(there is no CPU or PyTorch fallback for this plugin)")
        stamp = os.path.join(os.path.dirname(path), "pytorches_plugin_b200.built_from")
        if os.path.exists(stamp):  # written by the build: the digest of the sources the library came from
            from .build import source_digest

            with open(stamp) as f:
                if f.read().strip() != source_digest():
                    raise RuntimeError(f"{path} was built from other sources than the ones beside it: "
                                       "rebuild it with `python -m pytorches_b200.build`")
        _PLUGIN = Plugin(path)
    return _PLUGIN
