"""Generates tests/golden/shipped_wide.npz: tokens of the reference's SHIPPED sampler (the
unmodified sampler.cpp with its std::sort, Sampler::sample<float> on the exact upcast of the
16-bit logits) on rows of the benchmark configurations, for the tie-class comparison of
tests/test_gpu_parity_wide.py. The order of equal probabilities after std::sort is
unspecified, so the shipped build may return another token than the tie-pinned oracle -- but
only one with the same logit value.

Run from the repository root where the reference checkout is available:
    make -f oracle/Makefile ref && python tests/golden/make_shipped_wide.py
"""
import hashlib
import json
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

import oracle  # noqa: E402
from executorch_b200 import workloads as W  # noqa: E402

CASES = [
    # key, config, row ids, seeds per row
    ("c2", "c2", [0], 256),
    ("c3", "c3", list(range(256)), 1),
    ("c4", "c4", list(range(16)) + list(range(2048, 2064)), 1),
    ("c5", "c5", list(range(64)), 2),
]


def case_inputs(name, ids, per_row):
    x = W.rows_numpy(name, ids)
    xs = np.repeat(x, per_row, axis=0)
    seeds = (np.repeat(np.asarray(ids, dtype=np.uint64), per_row) * 1000
             + np.tile(np.arange(per_row, dtype=np.uint64), len(ids)) + 1)
    return x, xs, seeds


def main():
    shipped, stable = oracle.Reference(False), oracle.Reference(True)
    out, meta = {}, []
    threads = min(16, os.cpu_count() or 1)
    for key, name, ids, per_row in CASES:
        cfg = W.CONFIGS[name]
        x, xs, seeds = case_inputs(name, ids, per_row)
        tok = shipped.sample_rows(xs, cfg.temperature, cfg.topp, seeds, dtype=cfg.dtype, threads=threads)
        pinned = stable.sample_rows(xs, cfg.temperature, cfg.topp, seeds, dtype=cfg.dtype, threads=threads)
        out[key + "_shipped"] = tok
        meta.append(dict(key=key, name=name, row_ids=ids, per_row=per_row, temperature=cfg.temperature,
                         topp=cfg.topp, sha256=hashlib.sha256(x.tobytes()).hexdigest(),
                         shipped_equals_pinned=float((tok == pinned).mean())))
        print(key, "shipped == tie-pinned on", float((tok == pinned).mean()))
    out["meta"] = np.frombuffer(json.dumps(meta).encode(), dtype=np.uint8)
    path = os.path.join(ROOT, "tests", "golden", "shipped_wide.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
