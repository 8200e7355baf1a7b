"""Times the benchmark configurations on the CPU oracle (test infrastructure, not part of the product).

The oracle is a C++ restatement of the reference's CPU plugin; this script runs the same op sequences
``python -m pytorches_b200.configs`` issues to the B200 plugin against it, on this host's cores, so
that a CPU figure can stand beside each GPU figure. It is a reported baseline, not a target.

Usage:  python tests/cpu_configs.py [--config 1,3,4,4t] [--iters 3]
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import time

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from pytorches_b200.abi import Plugin  # noqa: E402
from pytorches_b200.configs import config1, config3_sharded, config4  # noqa: E402
from pytorches_b200.core import Device  # noqa: E402
from pytorches_b200.replay import Recorder, algorithmic_bytes  # noqa: E402

ORACLE_SO = os.path.join(ROOT, "oracle", "_build", "pytorches_plugin_cpuref.so")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", default="1,3,4,4t")
    ap.add_argument("--iters", type=int, default=3)
    args = ap.parse_args()
    makers = {"1": ("config 1", config1), "3": ("config 3", lambda d: config3_sharded(d, 0, 1)),
              "4": ("config 4, contiguous X", lambda d: config4(d, False)), "4t": ("config 4, transposed X", lambda d: config4(d, True))}
    oracle = Plugin(ORACLE_SO)
    for key in args.config.split(","):
        title, make = makers[key]
        rec = Recorder(oracle)  # only to count the algorithmic bytes of a step
        dev = Device(rec, 0)
        step = make(dev)
        step()
        rec.start()
        keep = step()
        counted = rec.finish(0)
        del keep
        times = []
        for _ in range(args.iters):
            t = time.perf_counter()
            step()
            times.append((time.perf_counter() - t) * 1e3)
        ms = statistics.median(times)
        nbytes = algorithmic_bytes(counted)
        print(json.dumps({"config": title, "plugin": "cpu oracle (C++ restatement of the reference CPU plugin)", "threads": os.cpu_count(),
                          "ops_per_step": counted.executes, "algorithmic_bytes": nbytes, "ms": round(ms, 3), "GB/s": round(nbytes / (ms * 1e-3) / 1e9, 2)}))
        sys.stdout.flush()


if __name__ == "__main__":
    main()
