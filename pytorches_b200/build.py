"""Builds ``pytorches_plugin_b200.so`` (and its manifest) in place, next to the sources in ``csrc/``.

Kernels are compiled offline to sm_100a machine code (no PTX JIT at load time). Flags that the
results depend on: ``-fmad=false`` (no multiply-add contraction: the reference CPU plugin never
contracts, FMA appears only where the code writes it), IEEE division and square root, no
flush-to-zero. The CUDA runtime is linked statically; it loads the driver lazily, so the library
loads on machines without a GPU and then reports zero devices.

Usage:  python -m pytorches_b200.build [--force] [--verbose]
"""

from __future__ import annotations

import json
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
ROOT = os.path.dirname(HERE)
SOURCES = ["plugin.cu", "ew.cu", "reduce.cu"]
HEADERS = ["common.cuh", "vecmath.cuh",
           os.path.join(ROOT, "include", "pytorches_plugin_abi.h"), os.path.join(ROOT, "include", "pytorches_b200_ext.h")]
OUT = os.path.join(CSRC, "pytorches_plugin_b200.so")
MANIFEST = os.path.join(CSRC, "pytorches_plugin_b200.json")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-fmad=false", "-prec-div=true", "-prec-sqrt=true", "-ftz=false",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "-cudart", "static",
]


def nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found: the B200 plugin cannot be built")
    return exe


STAMP = os.path.join(CSRC, "pytorches_plugin_b200.built_from")


def source_digest() -> str:
    """SHA-256 over everything the library is compiled from (sources, headers, flags). ``build`` records
    it beside the library and ``pytorches_b200.load_plugin`` refuses a library whose record differs
    from the sources next to it: a stale build would otherwise be measured and tested in their place."""
    import hashlib

    h = hashlib.sha256(" ".join(NVCC_FLAGS).encode())
    hdrs = [x if os.path.isabs(x) else os.path.join(CSRC, x) for x in HEADERS]
    for path in [os.path.join(CSRC, x) for x in SOURCES] + hdrs:
        with open(path, "rb") as f:
            h.update(os.path.basename(path).encode() + b"\0" + f.read())
    return h.hexdigest()


def _stale(target: str, deps: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    hdrs = [h if os.path.isabs(h) else os.path.join(CSRC, h) for h in HEADERS]
    objs = []
    jobs = []
    for src in SOURCES:
        s = os.path.join(CSRC, src)
        o = os.path.join(CSRC, src.replace(".cu", ".o"))
        objs.append(o)
        if force or _stale(o, [s, __file__] + hdrs):
            cmd = [nvcc(), *NVCC_FLAGS, "-c", s, "-o", o] + (["-Xptxas", "-v"] if verbose else [])
            jobs.append(cmd)

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"{' '.join(cmd)}\n{r.stdout}\n{r.stderr}")
        return r.stderr

    with ThreadPoolExecutor(max_workers=len(SOURCES)) as ex:
        for log in ex.map(run, jobs):
            if verbose and log:
                print(log, file=sys.stderr)
    if force or jobs or _stale(OUT, objs):
        # Export only the C ABI: the entry symbol and the extension entry points.
        run([nvcc(), *NVCC_FLAGS, "-shared", "-o", OUT, *objs])
    # Manifest next to the library (docs/plugin-abi.md:64-66; keys name, vendor, abi, os, arch).
    with open(MANIFEST, "w") as f:
        json.dump({"name": "b200", "vendor": "nvidia", "abi": 4, "os": "linux", "arch": "x86_64"}, f, indent=2)
        f.write("\n")
    with open(STAMP, "w") as f:
        f.write(source_digest() + "\n")
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
