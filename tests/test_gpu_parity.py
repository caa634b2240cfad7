"""Parity of the CUDA sampler (called through the C ABI) with the CPU oracle and with the
tokens of the reference's own compiled sampler (tests/golden).

Bars: argmax bit-exact (lowest index on ties); top-p and multinomial tokens identical to the
oracle's for at least 99.99 % of (row, seed) draws, and any differing draw must have its coin
within 1e-5 of a boundary of the oracle's cumulative distribution."""
import ctypes as C
import os
import subprocess
import tempfile

import numpy as np
import pytest
import torch

from executorch_b200 import (Sampler, _lib, logits_to_token, sample_all_from_logits,
                             sample_from_logits, seeds_to_states)
from executorch_b200 import workloads as W

from parity import compare_with_oracle, gpu_sample, to_device

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_extension_is_loaded_and_refuses_old_devices(cuda_device):
    lib = _lib.load()
    assert lib.etb200_sampler_abi_version() == 1
    assert torch.cuda.get_device_capability(cuda_device)[0] >= 10


def test_device_expf_is_bit_identical_to_host_libm(cuda_device):
    out = os.path.join(tempfile.mkdtemp(prefix="etb200_hc_"), "libhc.so")
    subprocess.run(["g++", "-std=c++17", "-O2", "-ffp-contract=off", "-fPIC", "-shared",
                    os.path.join(ROOT, "tests", "host_check.cpp"), "-o", out], check=True)
    hc = C.CDLL(out)
    hc.hc_libm_expf.argtypes = [C.c_void_p, C.c_void_p, C.c_long]
    rng = np.random.default_rng(3)
    # random negatives over the whole range, a dense sweep of bit patterns, and the differences
    # x - max that bf16 logits scaled by 1/0.7 actually produce
    a = (-rng.random(2_000_000) * 104.5).astype(np.float32)
    b = np.arange(0x80000000, 0xC2D10000, 521, dtype=np.uint32).view(np.float32)
    bf = (np.arange(0, 1 << 16, dtype=np.uint32) << 16).view(np.float32)
    bf = bf[np.isfinite(bf)]
    c = (bf * np.float32(1 / 0.7)).astype(np.float32)
    c = (c - np.float32(c[np.isfinite(c)].max() * 0 + 7.0)).astype(np.float32)
    x = np.ascontiguousarray(np.concatenate([a, b, c[c <= 0], [0.0, -0.0, -np.inf]]).astype(np.float32))
    want = np.empty_like(x)
    hc.hc_libm_expf(x.ctypes.data, want.ctypes.data, len(x))
    xd = torch.from_numpy(x).to(cuda_device)
    yd = torch.empty_like(xd)
    _lib.check(_lib.load().etb200_selftest_expf(
        C.c_void_p(xd.data_ptr()), C.c_void_p(yd.data_ptr()), len(x),
        C.c_void_p(torch.cuda.current_stream().cuda_stream)))
    got = yd.cpu().numpy()
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), \
        f"{(got.view(np.uint32) != want.view(np.uint32)).sum()} of {len(x)} differ"


def test_reference_argmax_fixtures(cuda_device):
    # extension/llm/sampler/test/test_sampler.cpp:19-43
    g = np.random.default_rng(7)
    x = g.random((1, 32000), dtype=np.float32) * np.float32(0.999)
    x[0, 396] = 1.0
    s = Sampler(32000, 0.0, 0.9, 0, device=cuda_device)
    assert s.sample(torch.from_numpy(x).to(cuda_device)) == 396
    xh = torch.from_numpy(x).to(cuda_device).to(torch.float16).clamp(max=0.999)
    xh[0, 396] = 1.0
    assert s.sample(xh) == 396
    # rank-3 [1, 1, V] input as in the test, through sample_from_logits
    assert sample_from_logits(xh.reshape(1, 1, -1), s) == 396
    s.close()
    # extension/llm/runner/test/test_text_decoder_runner.cpp:83-140 and :95-116
    for dt in (torch.float32, torch.float16, torch.bfloat16):
        t = torch.tensor([[0.1, 0.2, 0.8, 0.4]], dtype=dt, device=cuda_device)
        assert logits_to_token(t, 0.0) == 2
        t3 = torch.tensor([[[0.9, 0.1, 0.1, 0.1], [0.1, 0.2, 0.8, 0.4]]], dtype=dt, device=cuda_device)
        assert logits_to_token(t3, 0.0) == 2  # last sequence position
        tok = logits_to_token(t, 1.0)  # :143-153, result in range
        assert 0 <= tok < 4
    # extension/llm/runner/test/test_text_llm_runner.cpp:656-715
    lg = torch.tensor([[0.1, 0.2, 0.3, 0.4]], device=cuda_device)
    assert logits_to_token(lg, 0.0) == 3
    lg[0, 3] = float("-inf")
    assert logits_to_token(lg, 0.0) == 2
    lg[0, 2] = float("-inf")
    assert logits_to_token(lg, 0.0) == 1


def test_argmax_edge_semantics(cuda_device, restatement):
    cases = [
        np.array([[1.0, 3.0, 3.0, 2.0, 3.0]], dtype=np.float32),
        np.array([[-0.0, 0.0, -1.0]], dtype=np.float32),
        np.array([[np.nan, 5.0, 7.0]], dtype=np.float32),
        np.array([[1.0, np.nan, 0.5]], dtype=np.float32),
        np.array([[-np.inf, -np.inf, -np.inf]], dtype=np.float32),
        np.array([[-np.inf, -5.0, -np.inf, -5.0]], dtype=np.float32),
    ]
    for x in cases:
        want = restatement.sample_rows(x, 0.0, 0.9, np.zeros(1, np.uint64))
        got = gpu_sample(x, "fp32", 0.0, 0.9, [0], cuda_device)
        assert np.array_equal(got, want), x
    # ties spread over many threads and tiles; bit-exact in every dtype incl. raw uint16
    rng = np.random.default_rng(5)
    for dtype in ("fp32", "bf16", "fp16"):
        v = rng.integers(-3, 4, size=(37, 10007)).astype(np.float32)
        x = v if dtype == "fp32" else (W.f32_to_bf16_bits(v) if dtype == "bf16"
                                        else v.astype(np.float16).view(np.uint16))
        seeds = np.arange(37, dtype=np.uint64)
        want = restatement.sample_rows(x, 0.0, 0.9, seeds, dtype=dtype)
        got, st = gpu_sample(x, dtype, 0.0, 0.9, seeds, cuda_device, return_states=True)
        assert np.array_equal(got, want)
        assert np.array_equal(st, seeds)  # greedy never advances the RNG
    u = rng.integers(0, 65536, size=(9, 5003)).astype(np.uint16)
    want = restatement.sample_rows(u, 0.0, 0.9, np.zeros(9, np.uint64), dtype="u16")
    s = Sampler(5003, 0.0, 0.9, 0, device=cuda_device)
    t = torch.from_numpy(u.view(np.int16)).to(cuda_device).view(torch.uint16)
    assert np.array_equal(s.sample_rows(t).cpu().numpy(), want)
    s.close()


def test_golden_small_cases(cuda_device, golden):
    z, meta = golden
    n = 0
    for m in meta:
        if m["kind"] != "small":
            continue
        x, seeds = z[m["key"] + "_x"], z[m["key"] + "_seeds"]
        for si, (t, p) in enumerate(m["settings"]):
            got = gpu_sample(x, m["dtype"], t, p, seeds, cuda_device)
            assert np.array_equal(got, z[f"{m['key']}_st{si}"]), (m["vocab"], m["dtype"], t, p)
            n += len(got)
    assert n >= 1000


def test_golden_workload_cases(cuda_device, golden):
    z, meta = golden
    for m in meta:
        if m["kind"] != "workload":
            continue
        cfg = W.CONFIGS[m["name"]]
        x = W.rows_numpy(m["name"], m["row_ids"])
        seeds = np.asarray(m["row_ids"], dtype=np.uint64)
        for si, (t, p) in enumerate(m["settings"]):
            got = gpu_sample(x, cfg.dtype, t, p, seeds, cuda_device)
            want = z[f"w_{m['name']}_st{si}"]
            assert np.array_equal(got, want), (m["name"], t, p, np.nonzero(got != want)[0][:8])


def _check(report, what):
    n, eq, tol, bad, rows = report
    assert bad == 0, f"{what}: {bad} tokens differ beyond the 1e-5 coin tolerance (rows {rows[:8]})"
    assert eq >= n * 0.9999 - 1e-9, f"{what}: only {eq}/{n} identical ({tol} tolerated)"
    return eq, n


def test_config1_fp32_three_settings(cuda_device, restatement):
    ids = list(range(1500))
    x = W.rows_numpy("c1", ids)
    seeds = np.asarray(ids, dtype=np.uint64)  # rng_seed = row index; row 0 draws coin 0
    for t, p in ((0.0, 0.9), (0.8, 1.0), (0.8, 0.9)):
        _check(compare_with_oracle(restatement, x, "fp32", t, p, seeds, cuda_device), f"c1 T={t} topp={p}")


def test_config3_bf16_rows_by_seeds(cuda_device, restatement):
    ids = list(range(256))
    x = W.rows_numpy("c3", ids)
    reps = 12
    xs = np.tile(x, (reps, 1))
    seeds = np.concatenate([np.asarray(ids, dtype=np.uint64) + np.uint64(1000 * k) for k in range(reps)])
    _check(compare_with_oracle(restatement, xs, "bf16", 0.7, 0.95, seeds, cuda_device), "c3 top-p")
    _check(compare_with_oracle(restatement, x, "bf16", 0.7, 0.9, seeds[:256], cuda_device), "c3 top-p 0.9")
    _check(compare_with_oracle(restatement, x, "bf16", 0.7, 1.0, seeds[:256], cuda_device), "c3 multinomial")
    _check(compare_with_oracle(restatement, x, "bf16", 0.0, 0.95, seeds[:256], cuda_device), "c3 argmax")


def test_config2_decode_loop_single_row(cuda_device, restatement, golden):
    z, _ = golden
    row = z["seq_x"]
    s = Sampler(len(row), 0.7, 0.9, 12345, device=cuda_device)
    t = to_device(row[None, :], "bf16", cuda_device)[0]
    got = [s.sample(t) for _ in range(64)]
    assert got == list(z["seq_tok"])
    # full-size row, state evolving across draws, against the oracle's sequence
    full = W.rows_numpy("c2", [0])
    want = restatement.sample_sequence(W.to_f32(full, "bf16")[0], 0.7, 0.9, 777, 200)
    s2 = Sampler(full.shape[1], 0.7, 0.9, 777, device=cuda_device)
    tf = to_device(full, "bf16", cuda_device)[0]
    got = [s2.sample(tf) for _ in range(200)]
    assert got == list(want)
    assert s2.rng_state == restatement.coins(777, 200)[1][-1]
    s.close()
    s2.close()


def test_config4_fp16_peaked_and_flat(cuda_device, restatement):
    ids = [0, 1, 2, 3, 2048, 2049, 2050, 2051]
    x = W.rows_numpy("c4", ids)
    seeds = np.asarray(ids, dtype=np.uint64)
    _check(compare_with_oracle(restatement, x, "fp16", 1.0, 0.9, seeds, cuda_device), "c4 top-p")
    _check(compare_with_oracle(restatement, x, "fp16", 1.0, 1.0, seeds, cuda_device), "c4 multinomial")
    _check(compare_with_oracle(restatement, x, "fp16", 0.0, 0.9, seeds, cuda_device), "c4 argmax")


def test_config5_bf16_v256000(cuda_device, restatement):
    ids = list(range(96))
    x = W.rows_numpy("c5", ids)
    xs = np.tile(x, (4, 1))
    seeds = np.concatenate([np.asarray(ids, dtype=np.uint64) + np.uint64(500 * k) for k in range(4)])
    _check(compare_with_oracle(restatement, xs, "bf16", 0.8, 0.9, seeds, cuda_device), "c5 top-p")
    _check(compare_with_oracle(restatement, x, "bf16", 0.8, 1.0, seeds[:96], cuda_device), "c5 multinomial")
    _check(compare_with_oracle(restatement, x, "bf16", 0.0, 0.9, seeds[:96], cuda_device), "c5 argmax")


def test_ragged_shapes_strides_and_alignment(cuda_device, restatement):
    rng = np.random.default_rng(11)
    for vocab in (2, 3, 7, 33, 511, 513, 4095, 4097, 8191, 12345):
        for dtype in ("fp32", "bf16", "fp16"):
            v = (2.5 * rng.standard_normal((6, vocab))).astype(np.float32)
            x = v if dtype == "fp32" else (W.f32_to_bf16_bits(v) if dtype == "bf16"
                                            else v.astype(np.float16).view(np.uint16))
            seeds = rng.integers(0, 2**63, size=6).astype(np.uint64)
            for t, p in ((0.0, 0.9), (0.9, 1.0), (0.9, 0.8)):
                want = restatement.sample_rows(x, t, p, seeds, dtype=dtype)
                got = gpu_sample(x, dtype, t, p, seeds, cuda_device)
                assert np.array_equal(got, want), (vocab, dtype, t, p)
    # rows that are a strided, misaligned view of a larger buffer
    vocab, rows, pitch = 1001, 5, 1024 + 3
    v = (2.0 * rng.standard_normal((rows, pitch))).astype(np.float32)
    for dtype, tdt in (("fp32", torch.float32), ("bf16", torch.bfloat16)):
        base = torch.from_numpy(v).to(cuda_device).to(tdt)
        view = base[:, 1:1 + vocab]  # starts 1 element off alignment, row pitch != vocab
        host = view.contiguous().cpu()
        xh = host.numpy() if dtype == "fp32" else host.view(torch.int16).numpy().view(np.uint16)
        seeds = np.arange(rows, dtype=np.uint64) + 3
        for t, p in ((0.0, 0.9), (1.0, 0.0), (1.0, 0.9)):
            s = Sampler(vocab, t, p, 0, device=cuda_device)
            got = s.sample_rows(view, seeds_to_states(seeds, cuda_device)).cpu().numpy()
            s.close()
            want = restatement.sample_rows(xh, t, p, seeds, dtype=dtype)
            assert np.array_equal(got, want), (dtype, t, p)


def test_degenerate_distributions(cuda_device, restatement):
    vocab = 3000
    seeds = np.array([0, 1, 2, 3, 4, 5, 6, 7], dtype=np.uint64)  # seed 0 draws coin 0 forever
    flat = np.zeros((8, vocab), dtype=np.float32)  # every probability equal: ties everywhere
    onehot = np.full((8, vocab), -30.0, dtype=np.float32)
    onehot[np.arange(8), np.arange(8) * 37] = 5.0
    masked = (np.random.default_rng(2).standard_normal((8, vocab))).astype(np.float32)
    masked[:, ::2] = -np.inf  # half the vocabulary masked out by a logit processor
    two = np.tile(np.array([[0.3, 0.30001]], dtype=np.float32), (8, 1))
    for name, x in (("flat", flat), ("onehot", onehot), ("masked", masked), ("two", two)):
        for t, p in ((1.0, 0.9), (1.0, 1.0), (0.5, 0.1), (1.0, 0.999), (-1.0, 0.9)):
            want = restatement.sample_rows(x, t, p, seeds)
            got = gpu_sample(x, "fp32", t, p, seeds, cuda_device)
            assert np.array_equal(got, want), (name, t, p)
        xb = W.f32_to_bf16_bits(x)
        want = restatement.sample_rows(xb, 1.0, 0.9, seeds, dtype="bf16")
        assert np.array_equal(gpu_sample(xb, "bf16", 1.0, 0.9, seeds, cuda_device), want), name


def test_nucleus_sizes_around_the_shared_memory_limit(cuda_device, restatement):
    """Rows whose nucleus is a plateau of n equal logits (every comparison a tie, so the
    index order decides) over a low background, for n on both sides of the 512 survivors that
    the shared-memory tail takes; top-p that cuts inside the plateau, top-p that needs all of
    it, and top-k below, at and above n."""
    rng = np.random.default_rng(23)
    vocab = 40_000
    sizes = (1, 2, 31, 500, 511, 512, 513, 520, 700, 1500)
    x = np.full((len(sizes), vocab), -14.0, dtype=np.float32)
    x += (0.01 * rng.standard_normal(x.shape)).astype(np.float32)
    for r, n in enumerate(sizes):
        where = rng.permutation(vocab)[:n]
        x[r, where] = 3.0
        x[r, where[: max(1, n // 7)]] = 3.25  # a second, higher plateau inside it
    seeds = rng.integers(0, 2**62, size=len(sizes)).astype(np.uint64)
    for dtype in ("fp32", "bf16"):
        xd = x if dtype == "fp32" else W.f32_to_bf16_bits(x)
        for t, p, k in ((1.0, 0.6, 0), (1.0, 0.97, 0), (1.0, 0.9999, 0), (0.7, 0.9, 0),
                        (1.0, 0.9, 400), (1.0, 0.9, 512), (1.0, 0.9, 515), (1.0, 0.9, 5000)):
            want = restatement.sample_rows(xd, t, p, seeds, dtype=dtype, topk=k, threads=8)
            got = gpu_sample(xd, dtype, t, p, seeds, cuda_device, topk=k)
            assert np.array_equal(got, want), (dtype, t, p, k, np.nonzero(got != want)[0][:8])


def test_mixed_batch_larger_than_the_grid(cuda_device, restatement):
    """More rows than resident blocks, so every block samples several rows in turn and carries
    its candidate-floor guess from one row to the next; peaked, Zipf-shaped, flat and one-hot
    rows alternate so that the guess is wrong in both directions."""
    rng = np.random.default_rng(21)
    vocab, rows = 6000, 900
    x = np.empty((rows, vocab), dtype=np.float32)
    for r in range(rows):
        kind = r % 4
        if kind == 0:
            x[r] = -1.3 * np.log(1.0 + rng.permutation(vocab)) + 0.5 * rng.standard_normal(vocab)
        elif kind == 1:
            x[r] = 0.05 * rng.standard_normal(vocab)
        elif kind == 2:
            x[r] = rng.standard_normal(vocab)
            x[r, rng.integers(vocab)] = 25.0
        else:
            x[r] = 3.0 * rng.standard_normal(vocab)
    seeds = rng.integers(0, 2**62, size=rows).astype(np.uint64)
    for dtype in ("fp32", "bf16"):
        xd = x if dtype == "fp32" else W.f32_to_bf16_bits(x)
        for t, p, k in ((0.8, 0.9, 0), (1.0, 0.3, 0), (0.7, 0.99, 0), (0.9, 0.9, 25), (0.9, 0.9, 3000)):
            want = restatement.sample_rows(xd, t, p, seeds, dtype=dtype, topk=k, threads=8)
            got = gpu_sample(xd, dtype, t, p, seeds, cuda_device, topk=k)
            assert np.array_equal(got, want), (dtype, t, p, k, np.nonzero(got != want)[0][:8])


def test_vocabulary_beyond_one_compaction_segment(cuda_device, restatement):
    """A flat row of 300 000 fp16 logits: the nucleus holds ~270 000 tokens, so the candidate
    list spans several compaction segments and goes through the radix sort."""
    rng = np.random.default_rng(22)
    vocab = 300_000
    x = (0.05 * rng.standard_normal((2, vocab))).astype(np.float16).view(np.uint16)
    seeds = np.array([4, 5], dtype=np.uint64)
    for t, p, k in ((1.0, 0.9, 0), (1.0, 1.0, 0), (1.0, 0.9, 150_000)):
        want = restatement.sample_rows(x, t, p, seeds, dtype="fp16", topk=k)
        got = gpu_sample(x, "fp16", t, p, seeds, cuda_device, topk=k)
        assert np.array_equal(got, want), (t, p, k)


def test_mode_selection_setters_and_errors(cuda_device, restatement):
    x = W.rows_numpy("c1", [3, 4, 5], vocab=2048)
    t = torch.from_numpy(x).to(cuda_device)
    seeds = np.array([11, 12, 13], dtype=np.uint64)
    s = Sampler(2048, 0.8, 0.9, 0, device=cuda_device)
    a = s.sample_rows(t, seeds_to_states(seeds, cuda_device)).cpu().numpy()
    assert np.array_equal(a, restatement.sample_rows(x, 0.8, 0.9, seeds))
    s.set_temperature(-3.0)  # sampler.h:48-53: negative -> 0 -> greedy
    assert np.array_equal(s.sample_rows(t).cpu().numpy(), restatement.sample_rows(x, 0.0, 0.9, seeds))
    s.set_temperature(0.5)
    a = s.sample_rows(t, seeds_to_states(seeds, cuda_device)).cpu().numpy()
    assert np.array_equal(a, restatement.sample_rows(x, 0.5, 0.9, seeds))
    s.set_topk(2048)  # k >= vocab disables top-k (sampler.cpp:239)
    a = s.sample_rows(t, seeds_to_states(seeds, cuda_device)).cpu().numpy()
    assert np.array_equal(a, restatement.sample_rows(x, 0.5, 0.9, seeds))
    s.set_topk(5)  # top-k takes precedence over top-p (sampler.cpp:239-241)
    a = s.sample_rows(t, seeds_to_states(seeds, cuda_device)).cpu().numpy()
    assert np.array_equal(a, restatement.sample_rows(x, 0.5, 0.9, seeds, topk=5))
    s.set_topk(0)
    with pytest.raises(_lib.SamplerError) as e:
        s.sample_rows(t.to(torch.float64))
    assert e.value.code == _lib.NOT_SUPPORTED  # sample_from_logits aborts here (util.h:30-34)
    with pytest.raises(_lib.SamplerError) as e:
        s.sample_rows(t.view(torch.int32).to(torch.int16).view(torch.uint16)[:, :2048].contiguous(),
                      seeds_to_states(seeds, cuda_device))
    assert e.value.code == _lib.NOT_SUPPORTED  # raw uint16 with temperature != 0
    with pytest.raises(_lib.SamplerError) as e:
        s.sample_rows(t, None)  # several rows need per-row states
    assert e.value.code == _lib.INVALID_ARGUMENT
    with pytest.raises(ValueError):
        s.sample_rows(t[:, :100], seeds_to_states(seeds, cuda_device))
    s.close()
    # batched sample_from_logits over [B, S, V]: every batch row, last position
    s = Sampler(2048, 0.0, 0.9, 0, device=cuda_device)
    t3 = torch.stack([torch.flip(t, dims=[1]), t], dim=1)  # [3, 2, V]
    assert np.array_equal(sample_all_from_logits(t3, s).cpu().numpy(),
                          restatement.sample_rows(x, 0.0, 0.9, seeds))
    s.close()


def test_topk_reference_test_cases(cuda_device):
    """The five top-k tests of extension/llm/sampler/test/test_sampler.cpp:45-154."""
    # TestTopKRestrictsToCandidates
    s = Sampler(100, 1.0, 0.0, 42, device=cuda_device)
    s.set_topk(3)
    x = torch.full((100,), -10.0, device=cuda_device)
    x[7], x[13], x[42] = 5.0, 4.5, 4.0
    assert {s.sample(x) for _ in range(50)} <= {7, 13, 42}
    s.close()
    # TestTopKDisabledByZero
    s = Sampler(50, 1.0, 0.0, 7, device=cuda_device)
    s.set_topk(0)
    x = torch.full((50,), -10.0, device=cuda_device)
    x[11] = 20.0
    assert sum(s.sample(x) == 11 for _ in range(20)) >= 18
    s.close()
    # TestTopKWithFP16
    s = Sampler(50, 1.0, 0.0, 99, device=cuda_device)
    s.set_topk(2)
    x = torch.full((50,), -10.0, device=cuda_device, dtype=torch.float16)
    x[3], x[8] = 5.0, 4.5
    assert {s.sample(x) for _ in range(30)} <= {3, 8}
    s.close()
    # TestTopKEqualsOneIsArgmax
    s = Sampler(100, 1.0, 0.0, 123, device=cuda_device)
    s.set_topk(1)
    x = torch.rand(100, device=cuda_device)
    x[57] = 100.0
    assert all(s.sample(x) == 57 for _ in range(10))
    s.close()
    # TestTopKTakesPrecedenceOverTopP
    s = Sampler(100, 1.0, 0.99, 99, device=cuda_device)
    s.set_topk(2)
    x = torch.full((100,), -10.0, device=cuda_device)
    x[3], x[8], x[19] = 5.0, 4.5, 4.0
    assert {s.sample(x) for _ in range(50)} <= {3, 8}
    s.close()


def test_topk_parity(cuda_device, restatement, golden):
    z, meta = golden
    # tokens of the reference's own compiled sampler (fp32: no equal probabilities)
    for m in meta:
        if m["kind"] != "topk":
            continue
        x, seeds = z[m["key"] + "_x"], z[m["key"] + "_seeds"]
        for k in m["ks"]:
            got = gpu_sample(x, "fp32", m["temperature"], m["topp"], seeds, cuda_device, topk=k)
            assert np.array_equal(got, z[f"{m['key']}_k{k}"]), (m["vocab"], k)
    x = W.rows_numpy("c1", list(range(100)))
    got = gpu_sample(x, "fp32", 0.8, 0.9, np.arange(100, dtype=np.uint64), cuda_device, topk=40)
    assert np.array_equal(got, z["k_c1_k40"])
    # against the oracle (ties pinned to index order) on the benchmark-shaped rows
    for name, ids, ks in (("c1", range(300), (1, 40, 5000)), ("c3", range(64), (1, 50, 4000)),
                          ("c4", [0, 1, 2048, 2049], (8, 20000)), ("c5", range(16), (64,))):
        cfg = W.CONFIGS[name]
        x = W.rows_numpy(name, list(ids))
        seeds = np.asarray(list(ids), dtype=np.uint64) + 17
        for k in ks:
            want = restatement.sample_rows(x, cfg.temperature, cfg.topp, seeds, dtype=cfg.dtype, topk=k,
                                           threads=8)
            got = gpu_sample(x, cfg.dtype, cfg.temperature, cfg.topp, seeds, cuda_device, topk=k)
            assert np.array_equal(got, want), (name, k, np.nonzero(got != want)[0][:8])
    # low temperature: most exponentials underflow to 0, fewer than k entries are positive
    x = W.rows_numpy("c1", list(range(16)), vocab=4096)
    seeds = np.arange(16, dtype=np.uint64) + 3
    want = restatement.sample_rows(x, 0.05, 0.9, seeds, topk=3000)
    assert np.array_equal(gpu_sample(x, "fp32", 0.05, 0.9, seeds, cuda_device, topk=3000), want)


def test_pybind_module_drives_the_same_kernels(cuda_device, restatement):
    import sys
    libdir = os.path.join(ROOT, "executorch_b200", "lib")
    sys.path.insert(0, libdir)
    try:
        import _sampler_pybind as m
    finally:
        sys.path.remove(libdir)
    x = W.rows_numpy("c3", list(range(12)), vocab=20000)
    t = to_device(x, "bf16", cuda_device)
    seeds = np.arange(12, dtype=np.uint64) + 9
    states = seeds_to_states(seeds, cuda_device)
    out = torch.empty(12, dtype=torch.int64, device=cuda_device)
    s = m.Sampler(20000, 0.7, 0.9, 5, cuda_device.index)
    stream = torch.cuda.current_stream().cuda_stream
    s.sample_rows(t.data_ptr(), _lib.DTYPE_BFLOAT16, 12, t.stride(0), states.data_ptr(), out.data_ptr(), stream)
    torch.cuda.synchronize()
    assert np.array_equal(out.cpu().numpy(), restatement.sample_rows(x, 0.7, 0.9, seeds, dtype="bf16"))
    # single-row sample() with the sampler's own state (seed 5), three draws
    want = restatement.sample_sequence(W.to_f32(x[:1], "bf16")[0], 0.7, 0.9, 5, 3)
    got = [s.sample(t[0].data_ptr(), _lib.DTYPE_BFLOAT16, stream) for _ in range(3)]
    assert got == list(want)
    s.set_topk(7)
    s.rng_state = 77
    want = restatement.sample_rows(x[:1], 0.7, 0.9, np.array([77], dtype=np.uint64), dtype="bf16", topk=7)
    assert s.sample(t[0].data_ptr(), _lib.DTYPE_BFLOAT16, stream) == want[0]


def test_host_buffer_entry_matches_device_entry(cuda_device, restatement):
    x = W.rows_numpy("c3", list(range(16)), vocab=16384)
    seeds = np.arange(16, dtype=np.uint64) + 5
    s = Sampler(16384, 0.7, 0.95, 0, device=cuda_device)
    st = seeds.copy()
    got = s.sample_rows_host(x, st, dtype="bf16")
    want, wst = restatement.sample_rows(x, 0.7, 0.95, seeds, dtype="bf16", return_states=True)
    assert np.array_equal(got, want)
    assert np.array_equal(st, wst)  # states come back advanced
    s.set_temperature(0.0)
    assert np.array_equal(s.sample_rows_host(x, None, dtype="bf16"),
                          restatement.sample_rows(x, 0.0, 0.95, seeds, dtype="bf16"))
    s.close()


def test_host_buffer_entry_in_slices(cuda_device, restatement):
    """A batch large enough (100 rows, 12.8 MB) for the host-buffer entry point to copy in
    slices on its own stream while sampling earlier slices; ragged last slice; both the
    sampling and the greedy kernel; called twice so that the second call reuses the streams
    and events."""
    rows, vocab = 100, 32000
    x = W.rows_numpy("c1", list(range(rows)), vocab=vocab)
    seeds = np.arange(rows, dtype=np.uint64) * np.uint64(7919) + np.uint64(3)
    s = Sampler(vocab, 0.8, 0.9, 0, device=cuda_device)
    want, wst = restatement.sample_rows(x, 0.8, 0.9, seeds, dtype="fp32", return_states=True)
    for _ in range(2):
        st = seeds.copy()
        got = s.sample_rows_host(x, st, dtype="fp32")
        assert np.array_equal(got, want)
        assert np.array_equal(st, wst)
    s.set_temperature(0.0)
    assert np.array_equal(s.sample_rows_host(x, None, dtype="fp32"),
                          restatement.sample_rows(x, 0.0, 0.9, seeds, dtype="fp32"))
    s.close()


def test_chi_square_one_million_draws(cuda_device, restatement):
    """10^6 draws from one fixed config-3 row against the oracle's own nucleus distribution,
    top-p and multinomial; coins from 10^6 different seeds (a stride-0 batch)."""
    from scipy import stats
    row = W.rows_numpy("c3", [17])
    f32 = W.to_f32(row, "bf16")[0]
    n = 1_000_000
    seeds = (np.arange(n, dtype=np.uint64) * np.uint64(0x9E3779B97F4A7C15)) + np.uint64(12345)
    t = to_device(row, "bf16", cuda_device)
    for topp in (0.95, 1.0):
        s = Sampler(row.shape[1], 0.7, topp, 0, device=cuda_device)
        ids = s.sample_rows(t.expand(n, -1), seeds_to_states(seeds, cuda_device)).cpu().numpy()
        s.close()
        d = restatement.row_details(f32, 0.7, topp, 1)
        p = d["probs"].astype(np.float64)
        if topp < 1.0:
            cutoff = (1.0 - np.float32(topp)) / np.float32(len(p) - 1)
            cand = np.nonzero(d["probs"] >= cutoff)[0]
            order = cand[np.lexsort((cand, -d["probs"][cand]))][: d["last_idx"] + 1]
            assert np.isin(ids, order).all()  # nothing outside the nucleus is ever drawn
            q = np.zeros_like(p)
            q[order] = p[order]
        else:
            q = p
        q = q / q.sum()
        counts = np.bincount(ids, minlength=len(p)).astype(np.float64)
        expect = q * n
        big = expect >= 5
        obs = np.append(counts[big], counts[~big].sum())
        exp = np.append(expect[big], expect[~big].sum())
        if exp[-1] < 5:
            obs[-2] += obs[-1]; exp[-2] += exp[-1]; obs, exp = obs[:-1], exp[:-1]
        chi2 = ((obs - exp) ** 2 / exp).sum()
        pval = stats.chi2.sf(chi2, len(obs) - 1)
        assert pval > 1e-3, (topp, chi2, len(obs), pval)
    # a sample of the same draws, token by token, against the oracle
    k = 4096
    want = restatement.sample_rows(np.tile(row, (k, 1)), 0.7, 0.95, seeds[:k], dtype="bf16", threads=8)
    s = Sampler(row.shape[1], 0.7, 0.95, 0, device=cuda_device)
    ids = s.sample_rows(t.expand(k, -1), seeds_to_states(seeds[:k], cuda_device)).cpu().numpy()
    s.close()
    assert (ids == want).mean() >= 0.9999


def test_full_size_properties_on_device_generated_rows(cuda_device):
    """Size-independent properties at the benchmark's full sizes, inputs born on the device:
    determinism, greedy ids hold the row maximum, sampled ids lie inside an fp64 nucleus."""
    for name, rows in (("c3", 256), ("c5", 1024)):
        cfg = W.CONFIGS[name]
        x = W.rows_torch(name, 0, rows, cuda_device)
        seeds = np.arange(rows, dtype=np.uint64)
        s = Sampler(cfg.vocab, cfg.temperature, cfg.topp, 0, device=cuda_device)
        a = s.sample_rows(x, seeds_to_states(seeds, cuda_device))
        b = s.sample_rows(x, seeds_to_states(seeds, cuda_device))
        assert torch.equal(a, b)
        assert int(a.min()) >= 0 and int(a.max()) < cfg.vocab
        # a drawn token is never rarer than the probability where an fp64 nucleus ends
        p = torch.softmax(x.double() / cfg.temperature, dim=1)
        sp, _ = p.sort(dim=1, descending=True)
        edge = (sp.cumsum(dim=1) < cfg.topp + 1e-3).sum(dim=1).clamp(max=cfg.vocab - 1)
        p_edge = sp.gather(1, edge[:, None])[:, 0]
        p_tok = p.gather(1, a[:, None])[:, 0]
        assert bool((p_tok >= p_edge * (1 - 1e-6)).all())
        del p, sp
        s.set_temperature(0.0)
        g = s.sample_rows(x)
        assert torch.equal(x.gather(1, g[:, None])[:, 0], x.max(dim=1).values)
        # lowest index among equal maxima
        first = (x == x.max(dim=1, keepdim=True).values).float().argmax(dim=1)
        assert torch.equal(g, first)
        s.close()
        del x
