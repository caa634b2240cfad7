"""Host model of the cluster-per-row kernel's exact sequential sum (cluster_math.cuh): chunks
summarised from an inexact prefix estimate, then one walk over the event chunks. Whatever the
estimate, a decided sum must be the sequential float sum bit for bit; on the benchmark-shaped
rows the walk must decide."""
import ctypes as C
import os
import subprocess
import tempfile

import numpy as np
import pytest

from executorch_b200 import workloads as W

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
EV_CAP = 512


@pytest.fixture(scope="module")
def hc():
    out = os.path.join(tempfile.mkdtemp(prefix="etb200_hcc_"), "libhcc.so")
    subprocess.run(["g++", "-std=c++17", "-O2", "-ffp-contract=off", "-fPIC", "-shared",
                    os.path.join(ROOT, "tests", "host_cluster_check.cpp"), "-o", out], check=True)
    lib = C.CDLL(out)
    lib.hc_cluster_sum.restype = C.c_int
    lib.hc_cluster_sum.argtypes = [C.c_void_p, C.c_long, C.c_int, C.c_int, C.c_float,
                                   C.POINTER(C.c_float), C.POINTER(C.c_long)]
    lib.hc_row_terms.restype = None
    lib.hc_row_terms.argtypes = [C.c_void_p, C.c_long, C.c_float, C.c_void_p]
    return lib


def _cluster_sum(hc, e, slices, perturb=0.0, ev_cap=EV_CAP):
    e = np.ascontiguousarray(e, dtype=np.float32)
    s = C.c_float(0)
    stats = (C.c_long * 5)()
    rc = hc.hc_cluster_sum(e.ctypes.data, len(e), slices, ev_cap, perturb, C.byref(s), stats)
    return rc, np.float32(s.value), list(stats)


def _seq(e):
    return np.cumsum(np.asarray(e, dtype=np.float32), dtype=np.float32)[-1]


def _terms(hc, x, inv_t):
    x = np.ascontiguousarray(x, dtype=np.float32)
    e = np.empty_like(x)
    hc.hc_row_terms(x.ctypes.data, len(x), inv_t, e.ctypes.data)
    return e


@pytest.mark.parametrize("name,slices,rows", [("c3", 8, 24), ("c5", 16, 8), ("c2", 8, 1)])
def test_benchmark_rows_are_decided_and_exact(hc, name, slices, rows):
    cfg = W.CONFIGS[name]
    x = W.to_f32(W.rows_numpy(name, list(range(rows))), cfg.dtype)
    worst = 0
    for r in range(rows):
        e = _terms(hc, x[r], np.float32(1.0) / np.float32(cfg.temperature))
        rc, s, st = _cluster_sum(hc, e, slices)
        assert rc == 1, (name, r, rc, st)
        assert s.view(np.uint32) == _seq(e).view(np.uint32), (name, r)
        worst = max(worst, st[0])
    assert worst <= EV_CAP // 2  # the kernel's list has room to spare on these shapes


def _adversarial(rng, kind, n):
    if kind == 0:   # descending: the largest terms first
        return np.sort(np.exp(rng.normal(0, 4, n) - 12).astype(np.float32))[::-1]
    if kind == 1:   # ascending: the sum creeps towards every power of two
        return np.sort(np.exp(rng.normal(0, 4, n) - 12).astype(np.float32))
    if kind == 2:   # constant
        return np.full(n, np.float32(rng.random() * 1e-3), dtype=np.float32)
    if kind == 3:   # powers of two: exact half-way terms everywhere
        return (2.0 ** rng.integers(-30, 1, n)).astype(np.float32)
    if kind == 4:   # zeros, subnormals, long runs of zeros (masked tokens)
        v = np.where(rng.random(n) < 0.7, 0, rng.random(n) * 2.0 ** rng.integers(-149, -100, n).astype(np.float64))
        v[: n // 3] = 0
        return v.astype(np.float32)
    if kind == 5:   # huge dynamic range with one dominant term
        v = np.exp(rng.normal(0, 20, n) - 60).astype(np.float32)
        v[rng.integers(0, n)] = 1.0
        return v
    if kind == 6:   # a masked row: mostly zeros
        v = np.zeros(n, dtype=np.float32)
        idx = rng.integers(0, n, 50)
        v[idx] = rng.random(50).astype(np.float32)
        return v
    return ((rng.permutation(n).astype(np.float64) + 1) ** -1.57 * np.exp(rng.normal(0, 0.7, n))).astype(np.float32)


def test_a_decided_sum_is_always_the_sequential_sum(hc):
    """Adversarial rows and deliberately wrong estimates: the walk may give up, never lie."""
    rng = np.random.default_rng(7)
    decided = 0
    for trial in range(160):
        n = int(rng.integers(1, 70000))
        e = _adversarial(rng, trial % 8, n)
        want = _seq(e)
        for slices, perturb in ((8, 0.0), (3, 0.0), (8, 3e-3), (8, -3e-3), (16, 0.02), (8, -0.3)):
            rc, s, _ = _cluster_sum(hc, e, slices, perturb)
            if rc == 1:
                decided += 1
                assert s.view(np.uint32) == want.view(np.uint32), (trial, n, slices, perturb)
    assert decided > 300
