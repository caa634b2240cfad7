"""Host model of the value-class walk (class_math.cuh): the running float sum over runs of equal
terms, advanced in closed form, must stop at the same copy with the same sum as the plain loop
of the reference's sample_topp (sampler.cpp:150-170)."""
import ctypes as C
import os
import subprocess
import tempfile

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def hcc():
    out = os.path.join(tempfile.mkdtemp(prefix="etb200_hcl_"), "libhcl.so")
    subprocess.run(["g++", "-std=c++17", "-O2", "-ffp-contract=off", "-fPIC", "-shared",
                    os.path.join(ROOT, "tests", "host_class_check.cpp"), "-o", out], check=True)
    lib = C.CDLL(out)
    for name in ("hcc_brute", "hcc_walk"):
        getattr(lib, name).restype = C.c_int
    lib.hcc_brute.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_float, C.POINTER(C.c_float),
                              C.POINTER(C.c_long)]
    lib.hcc_walk.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_float, C.c_int, C.c_int,
                             C.POINTER(C.c_float), C.POINTER(C.c_long), C.POINTER(C.c_long)]
    lib.hcc_key.restype = C.c_uint32
    lib.hcc_key.argtypes = [C.c_uint32]
    lib.hcc_pattern.restype = C.c_uint32
    lib.hcc_pattern.argtypes = [C.c_uint32]
    return lib


def _both(hcc, p, cnt, thr, threads=8, per_thread=4):
    p = np.ascontiguousarray(p, dtype=np.float32)
    cnt = np.ascontiguousarray(cnt, dtype=np.int32)
    c0, c1 = C.c_float(0), C.c_float(0)
    k0, k1, rounds = C.c_long(0), C.c_long(0), C.c_long(0)
    f0 = hcc.hcc_brute(p.ctypes.data, cnt.ctypes.data, len(p), thr, C.byref(c0), C.byref(k0))
    f1 = hcc.hcc_walk(p.ctypes.data, cnt.ctypes.data, len(p), thr, threads, per_thread,
                      C.byref(c1), C.byref(k1), C.byref(rounds))
    a = (f0, np.float32(c0.value).view(np.uint32), k0.value)
    b = (f1, np.float32(c1.value).view(np.uint32), k1.value)
    return a, b, rounds.value


def _classes(rng, kind, n):
    if kind == 0:    # a flat row: almost equal probabilities, many copies each
        p = np.sort((1.0 / 150000) * np.exp(rng.normal(0, 0.05, n)))[::-1]
        cnt = rng.integers(0, 40, n)
    elif kind == 1:  # a peaked row
        p = np.sort(np.exp(rng.normal(0, 1, n)))[::-1]
        p[0] = np.exp(12.0)
        p = p / (p.sum() * 20)
        cnt = rng.integers(0, 30, n)
        cnt[0] = 1
    elif kind == 2:  # powers of two: exact half-way terms in many binades
        p = np.sort(2.0 ** rng.integers(-30, -3, n).astype(np.float64))[::-1]
        cnt = rng.integers(0, 9, n)
    elif kind == 3:  # one class holding everything (a constant row)
        p = np.array([rng.random() * 1e-5] * n)
        cnt = np.zeros(n, dtype=np.int64)
        cnt[rng.integers(0, n)] = int(rng.integers(1, 250000))
    elif kind == 4:  # 1.5 * 2^k: ties whose parity matters on the first copy
        p = np.sort(1.5 * 2.0 ** rng.integers(-28, -6, n).astype(np.float64))[::-1]
        cnt = rng.integers(0, 200, n)
    else:            # zeros and subnormals at the end of the list
        p = np.sort(np.concatenate([rng.random(n // 2) * 1e-3, rng.random(n - n // 2) * 1e-42]))[::-1]
        cnt = rng.integers(0, 5, n)
    return p.astype(np.float32), cnt.astype(np.int32)


def test_walk_matches_the_plain_loop(hcc):
    rng = np.random.default_rng(11)
    hits = 0
    for trial in range(240):
        n = int(rng.integers(1, 3000))
        p, cnt = _classes(rng, trial % 6, n)
        total = float(np.sum(p.astype(np.float64) * cnt))
        for frac in (0.0, 1e-4, 0.3, 0.9, 0.999, 1.0, 1.5):
            thr = np.float32(total * frac)
            a, b, _ = _both(hcc, p, cnt, thr, threads=int(rng.integers(1, 40)),
                            per_thread=int(rng.integers(1, 6)))
            assert a == b, (trial, n, frac, a, b)
            hits += a[0]
    assert hits > 600


def test_thresholds_on_the_trajectory_itself(hcc):
    """A threshold equal to a partial sum must stop one copy later (strict '>')."""
    rng = np.random.default_rng(5)
    for trial in range(60):
        n = int(rng.integers(2, 400))
        p, cnt = _classes(rng, trial % 6, n)
        seq = np.repeat(p, cnt)
        if len(seq) < 2:
            continue
        traj = np.cumsum(seq, dtype=np.float32)   # numpy accumulates sequentially in float32
        for k in rng.integers(0, len(traj), 6):
            a, b, _ = _both(hcc, p, cnt, traj[k])
            assert a == b, (trial, k, a, b)


def test_rounds_stay_few_on_a_flat_row(hcc):
    rng = np.random.default_rng(3)
    p, cnt = _classes(rng, 0, 16000)
    total = float(np.sum(p.astype(np.float64) * cnt))
    a, b, rounds = _both(hcc, p, cnt, np.float32(0.9 * total), threads=512, per_thread=4)
    assert a == b
    assert rounds <= 8 + 30   # one per tile plus one per binade crossing


def test_key_order(hcc):
    pats = np.arange(0, 65536, dtype=np.uint32)
    keys = np.array([hcc.hcc_key(int(x)) for x in pats[::7]], dtype=np.uint32)
    back = np.array([hcc.hcc_pattern(int(k)) for k in keys], dtype=np.uint32)
    assert (back == pats[::7]).all()
    vals = pats[::7].astype(np.uint16).view(np.float16).astype(np.float64)
    ok = np.isfinite(vals)
    order = np.argsort(keys[ok], kind="stable")
    assert (np.diff(vals[ok][order]) >= 0).all()


def test_runs_as_long_as_the_largest_vocabulary(hcc):
    """A few classes of up to 524 288 copies (the tail's vocabulary limit): products of count and
    increment beyond 32 bits, sums that cross many binades inside one run, thresholds of zero and
    beyond the total."""
    rng = np.random.default_rng(13)
    for trial in range(40):
        n = int(rng.integers(1, 6))
        p = np.sort(rng.choice([1.9e-6, 3e-7, 2.0 ** -20, 1.5 * 2.0 ** -19, 7.3e-3, 1e-38, 3e-41], n))[::-1]
        cnt = rng.integers(1, 524_289, n)
        p32, c32 = p.astype(np.float32), cnt.astype(np.int32)
        total = float(np.sum(p32.astype(np.float64) * c32))
        for thr in (0.0, total * 0.37, total * 0.999, total * 2.0 + 1e-30):
            a, b, _ = _both(hcc, p32, c32, np.float32(thr), threads=int(rng.integers(1, 8)), per_thread=4)
            assert a == b, (trial, p32, c32, thr, a, b)
