"""16-bit rows with a LONG nucleus (tens of thousands of tokens pass the cutoff crop of
sampler.cpp:136-143): the CUDA sampler takes its value-class tail for them (no candidate list, no
sort). Tokens must be identical to the oracle's, which sorts the candidates as the reference does
(equal probabilities by index)."""
import numpy as np
import pytest
import torch

from executorch_b200 import Sampler, seeds_to_states
from executorch_b200 import workloads as W

from parity import gpu_sample

pytestmark = pytest.mark.gpu


def _bits(v, dtype):
    return W.f32_to_bf16_bits(v) if dtype == "bf16" else v.astype(np.float16).view(np.uint16)


def _rows(rng, kind, vocab):
    if kind == "flat":
        return (0.05 * rng.standard_normal(vocab)).astype(np.float32)
    if kind == "peaked":
        v = rng.standard_normal(vocab).astype(np.float32)
        hot = rng.choice(vocab, 5, replace=False)
        v[hot[0]] = 12.0
        v[hot[1:]] = 8.0
        return v
    if kind == "quantised":   # few distinct values: classes of thousands of tokens
        return (np.round(rng.standard_normal(vocab) * 4) / 4).astype(np.float32)
    if kind == "constant":    # one class holds the whole row
        return np.full(vocab, 1.25, dtype=np.float32)
    if kind == "masked":      # a logit processor masked most tokens
        v = (0.3 * rng.standard_normal(vocab)).astype(np.float32)
        v[rng.random(vocab) < 0.6] = -np.inf
        return v
    if kind == "signs":       # values around zero: both signs, zeros of both signs, subnormals
        v = (1e-4 * rng.standard_normal(vocab)).astype(np.float32)
        v[::17] = 0.0
        v[5::17] = -0.0
        return v
    raise ValueError(kind)


KINDS = ("flat", "peaked", "quantised", "constant", "masked", "signs")


@pytest.mark.parametrize("dtype", ["fp16", "bf16"])
def test_long_nucleus_rows_match_the_oracle(cuda_device, restatement, dtype):
    rng = np.random.default_rng(31)
    for vocab in (151_936, 50_001, 3_000):
        reps = 6
        x = np.stack([_bits(_rows(rng, k, vocab), dtype) for k in KINDS for _ in range(reps)])
        seeds = rng.integers(0, 2**62, size=len(x)).astype(np.uint64)
        for t, p in ((1.0, 0.9), (1.3, 0.5), (0.8, 0.999), (2.0, 0.05)):
            want = restatement.sample_rows(x, t, p, seeds, dtype=dtype, threads=16)
            got = gpu_sample(x, dtype, t, p, seeds, cuda_device)
            bad = np.nonzero(got != want)[0]
            assert len(bad) == 0, (dtype, vocab, t, p, [(int(r), KINDS[r // reps]) for r in bad[:8]])


def test_many_draws_on_one_flat_and_one_peaked_row(cuda_device, restatement):
    """The coin sweeps the whole cumulative distribution: every window of classes gets hits."""
    rng = np.random.default_rng(32)
    vocab = 151_936
    for kind in ("flat", "peaked"):
        row = _bits(_rows(rng, kind, vocab), "fp16")
        x = np.tile(row, (512, 1))
        seeds = rng.integers(0, 2**62, size=512).astype(np.uint64)
        want = restatement.sample_rows(x, 1.0, 0.9, seeds, dtype="fp16", threads=16)
        got = gpu_sample(x, "fp16", 1.0, 0.9, seeds, cuda_device)
        assert np.array_equal(got, want), (kind, np.nonzero(got != want)[0][:8])


def test_misaligned_strided_view(cuda_device, restatement):
    rng = np.random.default_rng(33)
    vocab, rows, pitch = 40_001, 6, 40_960 + 3
    v = (0.05 * rng.standard_normal((rows, pitch))).astype(np.float32)
    for dtype, tdt in (("fp16", torch.float16), ("bf16", torch.bfloat16)):
        base = torch.from_numpy(v).to(cuda_device).to(tdt)
        view = base[:, 1:1 + vocab]
        xh = view.contiguous().cpu().view(torch.int16).numpy().view(np.uint16)
        seeds = np.arange(rows, dtype=np.uint64) + 9
        s = Sampler(vocab, 1.0, 0.9, 0, device=cuda_device)
        got = s.sample_rows(view, seeds_to_states(seeds, cuda_device)).cpu().numpy()
        s.close()
        want = restatement.sample_rows(xh, 1.0, 0.9, seeds, dtype=dtype)
        assert np.array_equal(got, want), dtype


@pytest.mark.parametrize("dtype", ["fp16", "bf16"])
def test_rows_with_their_own_settings_and_a_multiply(cuda_device, restatement, dtype):
    """The extended entry point: every row its own temperature / top-p, a multiply processor folded
    into the reads; long and short nuclei, greedy and multinomial rows mixed in one launch."""
    rng = np.random.default_rng(34)
    vocab, rows = 60_000, 40
    kinds = [KINDS[r % len(KINDS)] for r in range(rows)]
    x = np.stack([_bits(_rows(rng, k, vocab), dtype) for k in kinds])
    temps = rng.choice([0.0, 0.7, 1.0, 1.5], size=rows).astype(np.float32)
    topps = rng.choice([0.5, 0.9, 0.97, 1.0], size=rows).astype(np.float32)
    seeds = rng.integers(1, 2**62, size=rows).astype(np.uint64)
    scale = 0.5
    # the multiply works in place on the stored type: the product is rounded to it
    with np.errstate(invalid="ignore"):
        xs = _bits(W.to_f32(x, dtype) * np.float32(scale), dtype)
    want = np.array([restatement.sample_rows(xs[r:r + 1], float(temps[r]), float(topps[r]), seeds[r:r + 1],
                                             dtype=dtype)[0] for r in range(rows)])
    s = Sampler(vocab, 0.8, 0.9, 0, device=cuda_device)
    try:
        t = torch.from_numpy(np.ascontiguousarray(x).view(np.int16)).to(cuda_device)
        t = t.view(torch.bfloat16 if dtype == "bf16" else torch.float16)
        ids = s.sample_rows_ex(t, seeds_to_states(seeds, cuda_device),
                               temperature=torch.from_numpy(temps).to(cuda_device),
                               topp=torch.from_numpy(topps).to(cuda_device), scale=scale)
        torch.cuda.synchronize()
        got = ids.cpu().numpy()
        assert np.array_equal(got, want), [(int(r), kinds[r], float(temps[r]), float(topps[r]))
                                            for r in np.nonzero(got != want)[0][:8]]
        assert s.status == 0
    finally:
        s.close()


def test_more_long_rows_per_block_than_pending_records(cuda_device, restatement):
    """2 400 flat rows: every block meets more long-nucleus rows than the eight it records before it
    runs their tails, so the record list is flushed in the middle of the row loop."""
    rng = np.random.default_rng(35)
    vocab, rows = 40_001, 2_400
    base = np.stack([_bits(_rows(rng, "flat", vocab), "bf16") for _ in range(16)])
    x = np.tile(base, (rows // 16, 1))
    x[::7] = _bits(_rows(rng, "peaked", vocab), "bf16")  # rows that keep the sorted path in between
    seeds = rng.integers(0, 2**62, size=rows).astype(np.uint64)
    want = restatement.sample_rows(x, 1.0, 0.9, seeds, dtype="bf16", threads=16)
    got = gpu_sample(x, "bf16", 1.0, 0.9, seeds, cuda_device)
    assert np.array_equal(got, want), np.nonzero(got != want)[0][:8]


@pytest.mark.parametrize("dtype", ["fp16", "bf16"])
def test_random_long_nucleus_campaign(cuda_device, restatement, dtype):
    """1 200 random rows per dtype: random scale and shape of the logits (so that the nucleus is
    anything from a few thousand tokens to the whole row), random vocabulary size, temperature and
    top-p; a batch mixes rows that take the value-class tail with rows that keep the sorted path."""
    rng = np.random.default_rng(36 if dtype == "fp16" else 37)
    for batch in range(6):
        vocab = int(rng.integers(33_000, 90_000))
        rows = 200
        v = np.empty((rows, vocab), dtype=np.float32)
        for r in range(rows):
            kind = r % 5
            if kind == 0:      # nearly uniform
                v[r] = rng.uniform(0.005, 0.3) * rng.standard_normal(vocab)
            elif kind == 1:    # unit normal with a few hot tokens
                v[r] = rng.standard_normal(vocab)
                v[r, rng.integers(0, vocab, 3)] = rng.uniform(4, 14)
            elif kind == 2:    # heavy duplicates: logits on a coarse grid
                step = rng.choice([0.125, 0.25, 0.5])
                v[r] = np.round(rng.standard_normal(vocab) / step) * step
            elif kind == 3:    # Zipf-shaped: usually a short nucleus, the sorted path
                v[r] = -1.1 * np.log(1.0 + rng.permutation(vocab)) + 0.5 * rng.standard_normal(vocab)
            else:              # offset far from zero, both signs in different rows
                v[r] = rng.choice([-30.0, 30.0]) + rng.uniform(0.02, 1.5) * rng.standard_normal(vocab)
        x = _bits(v, dtype)
        seeds = rng.integers(0, 2**62, size=rows).astype(np.uint64)
        t = float(rng.choice([0.6, 1.0, 1.7, 3.0]))
        p = float(rng.choice([0.3, 0.8, 0.9, 0.97, 0.999]))
        want = restatement.sample_rows(x, t, p, seeds, dtype=dtype, threads=16)
        got = gpu_sample(x, dtype, t, p, seeds, cuda_device)
        bad = np.nonzero(got != want)[0]
        assert len(bad) == 0, (dtype, batch, vocab, t, p, [(int(r), int(r) % 5) for r in bad[:8]])
