"""Generates tests/golden/sampler_golden.npz by running the reference's own, unmodified
sampler.cpp (compiled into oracle/_ref by oracle/Makefile) on seeded inputs.

Run from the repository root where the reference checkout is available:
    make -f oracle/Makefile ref && python tests/golden/make_golden.py

Stored per case: the settings, the tokens of the tie-pinned build (`tok_stable`) and of
the shipped std::sort build (`tok_shipped`). Small cases store their inputs; cases shaped
like the benchmark configurations store a SHA-256 of the regenerated inputs instead.
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


def small_inputs(vocab, dtype, rows, seed):
    g = np.random.default_rng(seed)
    kind = seed % 3
    if kind == 0:
        x = 3.0 * g.standard_normal((rows, vocab), dtype=np.float32)
    elif kind == 1:
        x = (-1.2 * np.log(1.0 + g.permuted(np.tile(np.arange(vocab, dtype=np.float32), (rows, 1)), axis=1))
             + 0.5 * g.standard_normal((rows, vocab), dtype=np.float32)).astype(np.float32)
    else:
        x = 0.05 * g.standard_normal((rows, vocab), dtype=np.float32)
    if dtype == "bf16":
        return W.f32_to_bf16_bits(x)
    if dtype == "fp16":
        return x.astype(np.float16).view(np.uint16)
    return x


def main():
    stable, shipped = oracle.Reference(True), oracle.Reference(False)
    out, meta = {}, []
    settings = [(0.0, 0.9), (0.8, 1.0), (0.8, 0.9), (1.0, 0.5), (0.3, 0.99), (1.0, 0.0)]
    cid = 0
    for vocab in (5, 64, 1000, 4099):
        for dtype in ("fp32", "bf16", "fp16"):
            rows = 16
            x = small_inputs(vocab, dtype, rows, seed=1000 + cid)
            seeds = np.arange(rows, dtype=np.uint64) * 7919 + cid
            key = f"s{cid}"
            out[key + "_x"] = x
            out[key + "_seeds"] = seeds
            for si, (t, p) in enumerate(settings):
                out[f"{key}_st{si}"] = stable.sample_rows(x, t, p, seeds, dtype=dtype)
                out[f"{key}_sh{si}"] = shipped.sample_rows(x, t, p, seeds, dtype=dtype)
            meta.append(dict(key=key, kind="small", vocab=vocab, dtype=dtype, rows=rows,
                             settings=settings))
            cid += 1
    for name, ids in (("c1", list(range(200))), ("c3", list(range(32))),
                      ("c5", list(range(8))), ("c4", [0, 1, 2048, 2049])):
        cfg = W.CONFIGS[name]
        x = W.rows_numpy(name, ids)
        seeds = np.asarray(ids, dtype=np.uint64)
        key = f"w_{name}"
        sets = [(0.0, cfg.topp), (cfg.temperature, 1.0), (cfg.temperature, cfg.topp)]
        for si, (t, p) in enumerate(sets):
            out[f"{key}_st{si}"] = stable.sample_rows(x, t, p, seeds, dtype=cfg.dtype, threads=8)
            out[f"{key}_sh{si}"] = shipped.sample_rows(x, t, p, seeds, dtype=cfg.dtype, threads=8)
        meta.append(dict(key=key, kind="workload", name=name, row_ids=ids, settings=sets,
                         sha256=hashlib.sha256(x.tobytes()).hexdigest()))
    # top-k (sampler.cpp:72-120) on fp32 inputs, where no two probabilities are equal and the
    # unspecified tie order of std::partial_sort cannot matter
    for vocab, ks in ((64, (1, 3, 50)), (1000, (1, 40, 999)), (4099, (2, 100))):
        x = small_inputs(vocab, "fp32", 24, seed=2000 + vocab)
        seeds = np.arange(24, dtype=np.uint64) * 31 + 5
        key = f"k{vocab}"
        out[key + "_x"] = x
        out[key + "_seeds"] = seeds
        for k in ks:
            out[f"{key}_k{k}"] = shipped.sample_rows(x, 0.9, 0.9, seeds, dtype="fp32", topk=k)
        meta.append(dict(key=key, kind="topk", vocab=vocab, ks=list(ks), temperature=0.9, topp=0.9))
    x = W.rows_numpy("c1", list(range(100)))
    out["k_c1_k40"] = shipped.sample_rows(x, 0.8, 0.9, np.arange(100, dtype=np.uint64), dtype="fp32",
                                          topk=40, threads=8)
    # decode-loop usage: one sampler, evolving state, 64 draws from one row
    row = W.rows_numpy("c3", [5], vocab=8192)[0]
    out["seq_x"] = row
    out["seq_tok"] = stable.sample_sequence(row, 0.7, 0.9, 12345, 64, dtype="bf16")
    out["meta"] = np.frombuffer(json.dumps(meta).encode(), dtype=np.uint8)
    path = os.path.join(ROOT, "tests", "golden", "sampler_golden.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
