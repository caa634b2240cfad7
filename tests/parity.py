"""Helpers shared by the GPU parity tests: running the CUDA sampler through its Python
mirror (which goes through the C ABI) and classifying any token that differs from the
oracle's."""
from __future__ import annotations

import os

import numpy as np
import torch

from executorch_b200 import Sampler, seeds_to_states
from executorch_b200 import workloads as W

THREADS = max(1, min(32, os.cpu_count() or 1))


def to_device(x: np.ndarray, dtype: str, device) -> torch.Tensor:
    if dtype == "fp32":
        return torch.from_numpy(np.ascontiguousarray(x, dtype=np.float32)).to(device)
    t = torch.from_numpy(np.ascontiguousarray(x).view(np.int16)).to(device)
    return t.view(torch.bfloat16 if dtype == "bf16" else torch.float16)


def gpu_sample(x: np.ndarray, dtype: str, temperature: float, topp: float, seeds, device,
               return_states: bool = False, topk: int = 0):
    rows, vocab = x.shape
    s = Sampler(vocab, temperature, topp, 0, device=device)
    try:
        if topk:
            s.set_topk(topk)
        t = to_device(x, dtype, device)
        states = seeds_to_states(seeds, device)
        ids = s.sample_rows(t, states)
        torch.cuda.synchronize(device)
        out = ids.cpu().numpy()
        if return_states:
            return out, states.cpu().numpy().view(np.uint64)
        return out
    finally:
        s.close()


def mismatch_is_within_tolerance(restatement, row_f32: np.ndarray, temperature: float,
                                 topp: float, seed: int, gpu_token: int, tol: float = 1e-5) -> bool:
    """A differing token is tolerated only if the row's coin lies within `tol` of a boundary
    of the GPU token's slot in the oracle's own cumulative distribution (float64 sums of the
    oracle's float probabilities, in the oracle's order)."""
    d = restatement.row_details(row_f32, temperature, topp, seed)
    p = d["probs"].astype(np.float64)
    coin = float(d["coin"])
    if topp <= 0 or topp >= 1:
        cdf = np.cumsum(p)
        lo = cdf[gpu_token - 1] if gpu_token > 0 else 0.0
        hi = cdf[gpu_token]
        return lo - tol <= coin <= hi + tol
    cutoff = (1.0 - np.float32(topp)) / np.float32(len(p) - 1)
    cand = np.nonzero(d["probs"] >= cutoff)[0]
    order = cand[np.lexsort((cand, -d["probs"][cand]))]
    last = d["last_idx"]
    # allow the nucleus edge itself to move by one slot
    order = order[: last + 2]
    where = np.nonzero(order == gpu_token)[0]
    if len(where) == 0:
        return False
    cdf = np.cumsum(p[order])
    total = cdf[min(last, len(cdf) - 1)]
    j = int(where[0])
    lo = (cdf[j - 1] if j > 0 else 0.0) / total
    hi = cdf[j] / total
    return lo - tol <= coin <= hi + tol


def compare_with_oracle(restatement, x: np.ndarray, dtype: str, temperature: float, topp: float,
                        seeds, device):
    """Returns (n, n_equal, n_tolerated, n_bad, bad_rows)."""
    got = gpu_sample(x, dtype, temperature, topp, seeds, device)
    want = restatement.sample_rows(x, temperature, topp, np.asarray(seeds, dtype=np.uint64),
                                   dtype=dtype, threads=THREADS)
    diff = np.nonzero(got != want)[0]
    tolerated, bad = 0, []
    for r in diff:
        row = W.to_f32(x[r:r + 1], dtype)[0]
        if mismatch_is_within_tolerance(restatement, row, temperature, topp, int(seeds[r]), int(got[r])):
            tolerated += 1
        else:
            bad.append(int(r))
    return len(got), len(got) - len(diff), tolerated, len(bad), bad
