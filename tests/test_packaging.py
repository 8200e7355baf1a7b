"""The plugin is discoverable the way the reference discovers separately installed backends.

``crates/python/python/pytorches/_discover.py:22-44`` reads the ``pytorches.plugins`` entry points; each
value names a module, which is located (not imported) and whose directory is searched for
``pytorches_plugin_*`` libraries; ``crates/core/src/plugin/manifest.rs:40-60`` then checks the manifest
beside each library without loading it. These tests walk the same steps over this repository.
"""

import importlib.util
import json
import os
import pathlib
import platform
import tomllib

ROOT = pathlib.Path(__file__).resolve().parent.parent


def entry_points():
    with open(ROOT / "pyproject.toml", "rb") as f:
        return tomllib.load(f)["project"]["entry-points"]["pytorches.plugins"]


def test_entry_point_names_the_directory_that_holds_the_library():
    eps = entry_points()
    assert list(eps) == ["b200"]
    module = eps["b200"].split(":")[0].strip()
    spec = importlib.util.find_spec(module)  # _discover.py:28-31
    assert spec is not None
    dirs = [pathlib.Path(p) for p in (spec.submodule_search_locations or [])] or [pathlib.Path(spec.origin).parent]
    dirs = [d for d in dirs if d.is_dir()]
    assert dirs, "the entry point's module has no directory"
    libs = [f for d in dirs for f in os.listdir(d) if f.startswith("pytorches_plugin_") and f.endswith(".so")]
    assert libs == ["pytorches_plugin_b200.so"], "build the plugin first: python -m pytorches_b200.build"


def test_manifest_passes_the_loaders_first_gate():
    lib = ROOT / "pytorches_b200" / "csrc" / "pytorches_plugin_b200.so"
    manifest = lib.with_name(lib.stem.removeprefix("lib") + ".json")  # manifest.rs:56-59
    m = json.loads(manifest.read_text())
    assert m["name"] == "b200" and m["abi"] == 4  # manifest.rs:41-45: the ABI must equal the core's
    as_list = lambda v: [v] if isinstance(v, str) else list(v)  # manifest.rs:90-103: a string or a list of strings
    assert "linux" in as_list(m["os"])
    assert platform.machine() in as_list(m["arch"])
