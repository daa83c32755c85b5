"""Per-module device times of one of the benchmark networks: `python esp-dl_b200/profile_model.py yolo11n_640 --batch 512`.

Builds the network (seeded random weights, as bench.py does), runs it on cuda:0 and prints, from dl::Model's
per-module CUDA-event times (minimum of three passes), the time per operator kind and the slowest modules.
"""
import argparse
import collections
import os
import sys
import tempfile

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
import __graft_entry__ as entry  # noqa: E402

entry._package()
from espdl_b200 import model, zoo  # noqa: E402


def build(name):
    if name == "yolo11n_640":
        return zoo.yolo11n_640(os.path.join(ROOT, "tests", "golden", "yolo11n_640_topology.json"), seed=6)
    if name == "mobilenet_v2":
        return zoo.mobilenet_v2(seed=5)
    if name == "mbv2_block":
        return zoo.inverted_residual_block(seed=4)
    raise SystemExit(f"unknown network {name}")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("network", choices=["yolo11n_640", "mobilenet_v2", "mbv2_block"])
    ap.add_argument("--batch", type=int, default=512)
    ap.add_argument("--top", type=int, default=20)
    a = ap.parse_args()
    with tempfile.TemporaryDirectory() as tmp:
        path = os.path.join(tmp, a.network + ".espdl")
        build(a.network).save(path)
        m = model.Model(path, batch=a.batch)
    m.inputs[0].array[...] = np.random.default_rng(0).integers(-128, 128, size=m.inputs[0].shape, dtype=np.int8)
    m.run()
    best, rows = None, None
    for _ in range(3):
        rows = m.profile()
        t = [r[2] for r in rows]
        best = t if best is None else [min(x, y) for x, y in zip(best, t)]
    kind, count = collections.defaultdict(float), collections.Counter()
    for r, t in zip(rows, best):
        kind[r[1]] += t
        count[r[1]] += 1
    total = sum(best)
    print(f"{a.network} batch {a.batch}: {len(rows)} modules, {m.num_slice_views()} tensors as channel slices, "
          f"arena {m.arena_bytes / 1e6:.0f} MB, sum of module times {total / 1000:.2f} ms")
    for k, v in sorted(kind.items(), key=lambda kv: -kv[1]):
        print(f"  {k:20s} {count[k]:4d} x {v / 1000:8.2f} ms {100 * v / total:5.1f} %")
    print(f"slowest {a.top} modules:")
    for t, r in sorted(zip(best, rows), key=lambda x: -x[0])[:a.top]:
        print(f"  {r[3][:52]:52s} {r[1]:18s} {t:8.1f} us")
    m.close()


if __name__ == "__main__":
    main()
