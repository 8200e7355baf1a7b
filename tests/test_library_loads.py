"""CPU run: the built plugin loads without a GPU, exports every declared symbol, and reports no devices."""

import ctypes
import os
import re

import pytest

import pytorches_b200
from pytorches_b200 import abi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    """Function names declared in include/*.h (lines of the form `<type> name(args);` at top level)."""
    names = set()
    for fn in sorted(os.listdir(os.path.join(ROOT, "include"))):
        text = open(os.path.join(ROOT, "include", fn)).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        text = re.sub(r"typedef struct \w+ \{.*?\} \w+;", "", text, flags=re.S)
        for m in re.finditer(r"^[A-Za-z_][\w \*]*?\b(pytorches_\w+)\s*\(", text, flags=re.M):
            names.add(m.group(1))
    return names


@pytest.fixture(scope="module")
def built():
    if not os.path.exists(pytorches_b200.plugin_path()):
        from pytorches_b200.build import build

        build()
    return pytorches_b200.plugin_path()


def test_exports_every_declared_symbol(built):
    lib = ctypes.CDLL(built)
    declared = _declared_symbols()
    assert "pytorches_plugin_entry" in declared and "pytorches_b200_stream" in declared
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared in include/ but not exported"


def test_vtable_is_well_formed(built):
    p = abi.Plugin(built)  # applies the loader's ABI / struct_size checks
    assert p.name == "b200"
    assert p.vt.struct_size >= ctypes.sizeof(abi.PluginVTable)
    for code in [abi.op.NEG, abi.op.EXP, abi.op.LOG, abi.op.RELU, abi.op.TANH, abi.op.STEP, abi.op.ADD, abi.op.SUB, abi.op.MUL,
                 abi.op.DIV, abi.op.MATMUL, abi.op.SUM_AXIS, abi.op.COPY, abi.op.FILL, abi.op.RAND_NORMAL]:
        assert p.supports_op(code), f"required op {code} not advertised (docs/plugin-abi.md:176-188)"
    assert p.supports_op(abi.op.AXPY) and p.supports_op(abi.op.MAX_AXIS) and p.supports_op(abi.op.ARGMAX_AXIS)
    assert not p.supports_op(9999)


def test_no_gpu_means_no_devices_and_no_fallback(built):
    """Without a GPU the plugin reports zero devices quietly and every call fails with a status."""
    import torch

    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    p = abi.Plugin(built)
    assert p.device_count() == 0
    with pytest.raises(abi.PluginError):
        p.alloc(0, 16)
    assert p.execute_status(0, abi.op.FILL, [0], [], [abi.Arg(0, (1,), (1,))]) != abi.STATUS_OK


def test_manifest_matches(built):
    import json

    m = json.load(open(os.path.join(os.path.dirname(built), "pytorches_plugin_b200.json")))
    assert m["name"] == "b200" and m["abi"] == abi.ABI_VERSION


def test_a_library_built_from_other_sources_is_refused(built, monkeypatch):
    """The build records a digest of its sources beside the library; a library whose record does not match
    the sources next to it (somebody edited a kernel and forgot to rebuild) must not be loaded silently."""
    import pytorches_b200.build as build

    stamp = os.path.join(os.path.dirname(built), "pytorches_plugin_b200.built_from")
    if not os.path.exists(stamp):
        build.build()
    monkeypatch.setattr(pytorches_b200, "_PLUGIN", None)
    assert pytorches_b200.load_plugin().name == "b200"
    monkeypatch.setattr(pytorches_b200, "_PLUGIN", None)
    monkeypatch.setattr(build, "source_digest", lambda: "0" * 64)
    with pytest.raises(RuntimeError, match="rebuild"):
        pytorches_b200.load_plugin()
