"""The alternative sampling kernels -- a thread-block cluster per row plus a finishing kernel
(choice 2), one block per row with the estimate-guided exact sum (choice 3) -- must return the
tokens and advanced RNG states of the one-block-per-row kernel (choice 1), which in turn are
the oracle's. Shapes cover one and several slices per row, ragged ends, rows that the fast
kernels hand back (long nuclei, flat rows), fp16, repeated rows and the automatic choice."""
import numpy as np
import pytest
import torch

from executorch_b200 import Sampler, seeds_to_states
from executorch_b200 import workloads as W

from parity import THREADS, to_device

pytestmark = pytest.mark.gpu


def _run(x, dtype, temperature, topp, seeds, device, choice, stride0=False):
    rows, vocab = x.shape
    s = Sampler(vocab, temperature, topp, 0, device=device)
    try:
        s.set_kernel_choice(choice)
        t = to_device(x, dtype, device)
        if stride0:
            t = t[:1].expand(rows, vocab)
        states = seeds_to_states(seeds, device)
        ids = s.sample_rows(t, states)
        torch.cuda.synchronize(device)
        return ids.cpu().numpy(), states.cpu().numpy().view(np.uint64), s.last_retry_count
    finally:
        s.close()


CASES = [
    # name, rows, vocab, temperature, topp
    ("c3", 6, 300, 0.7, 0.95),
    ("c3", 5, 4099 // 8 * 8, 0.7, 0.9),
    ("c3", 4, 16384, 0.7, 0.95),
    ("c3", 7, 16392, 1.0, 0.8),
    ("c3", 9, 33000, 0.7, 0.95),
    ("c3", 5, 100003, 0.5, 0.99),      # ragged last chunk, not a multiple of 8
    ("c3", 40, None, 0.7, 0.95),       # the headline shape
    ("c3", 12, None, 1.0, 0.5),        # long nuclei: the fast kernels hand rows back
    ("c2", 1, None, 0.7, 0.9),
    ("c5", 6, None, 0.8, 0.9),         # 16 slices per row
    ("c4", 2, 20000, 1.0, 0.9),        # fp16 (guided only; the cluster pair leaves it to kernel 1)
]


@pytest.mark.parametrize("choice", [2, 3])
@pytest.mark.parametrize("name,rows,vocab,temperature,topp", CASES)
def test_alternative_kernels_return_the_reference_tokens(cuda_device, restatement, choice, name, rows, vocab,
                                                         temperature, topp):
    cfg = W.CONFIGS[name]
    x = W.rows_numpy(name, list(range(rows)), vocab=vocab)
    seeds = (np.arange(rows, dtype=np.uint64) * 7919 + 1) % 1000003
    seeds[0] = 0  # a zero state draws coin 0 forever
    want = restatement.sample_rows(x, temperature, topp, seeds, dtype=cfg.dtype, threads=THREADS)
    base, base_states, _ = _run(x, cfg.dtype, temperature, topp, seeds, cuda_device, 1)
    got, states, retries = _run(x, cfg.dtype, temperature, topp, seeds, cuda_device, choice)
    assert np.array_equal(base, want)
    assert np.array_equal(got, want), (choice, name, np.nonzero(got != want)[0][:8])
    assert np.array_equal(states, base_states)
    assert 0 <= retries <= rows


def test_headline_rows_are_decided_by_the_fast_kernels(cuda_device):
    """On the headline shape the fast kernels hand back at most a few rows."""
    rows = 64
    x = W.rows_numpy("c3", list(range(rows)))
    seeds = np.arange(rows, dtype=np.uint64)
    for choice in (2, 3):
        _, _, retries = _run(x, "bf16", 0.7, 0.95, seeds, cuda_device, choice)
        assert retries <= rows // 8, (choice, retries)


def test_repeated_row_and_automatic_choice(cuda_device, restatement):
    """Stride 0 (one row, many states) through every kernel; a single long row takes the cluster
    pair automatically and matches the oracle's decode sequence."""
    x = W.rows_numpy("c2", [0])
    seeds = np.arange(24, dtype=np.uint64) + 5
    xs = np.repeat(x, len(seeds), axis=0)
    want = restatement.sample_rows(xs, 0.7, 0.9, seeds, dtype="bf16", threads=THREADS)
    for choice in (1, 2, 3):
        got, _, _ = _run(xs, "bf16", 0.7, 0.9, seeds, cuda_device, choice, stride0=True)
        assert np.array_equal(got, want), choice
    s = Sampler(x.shape[1], 0.7, 0.9, 12345, device=cuda_device)
    try:
        t = to_device(x, "bf16", cuda_device)
        got = [s.sample(t[0]) for _ in range(12)]
        n0 = s.launch_count
        s.sample(t[0])
        assert s.launch_count - n0 == 3  # cluster kernel, finishing kernel, the (empty) retry pass
    finally:
        s.close()
    want_seq = restatement.sample_sequence(W.to_f32(x, "bf16")[0], 0.7, 0.9, 12345, 12)
    assert got == [int(v) for v in want_seq]
