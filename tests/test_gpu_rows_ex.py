"""etb200_sampler_sample_rows_ex: a serving batch whose rows carry their own SamplingConfig
(llm_session.h:29-34) and whose logit processors -- mask, bias, multiply (logit_processor.h:
34-40) -- run on the device. Checked against the oracle run row by row on logits that were
processed on the host the way such processors process them (in place, in the logits' dtype).
The processor cases follow extension/llm/sampler/test/test_logit_processor.cpp:109-223 and
extension/llm/runner/test/test_text_llm_runner.cpp:656-715."""
import numpy as np
import pytest
import torch

from executorch_b200 import Sampler, seeds_to_states
from executorch_b200._lib import SamplerError
from executorch_b200 import workloads as W

from parity import to_device

pytestmark = pytest.mark.gpu


def _to_storage(v32, dtype):
    if dtype == "fp32":
        return v32.astype(np.float32)
    if dtype == "bf16":
        return W.f32_to_bf16_bits(v32)
    return v32.astype(np.float16).view(np.uint16)


def _host_process(x, dtype, edits_per_row, scale):
    """What the processors do to the stored logits: += bias (rounded to the dtype), then *= scale."""
    out = x.copy()
    for r, edits in enumerate(edits_per_row):
        for tid, bias in edits:
            if 0 <= tid < x.shape[1]:
                v = W.to_f32(out[r:r + 1, tid:tid + 1], dtype)[0, 0] + np.float32(bias)
                out[r, tid] = _to_storage(np.array([v], dtype=np.float32), dtype)[0]
    if scale != 1.0:
        with np.errstate(invalid="ignore"):
            out = _to_storage(W.to_f32(out, dtype) * np.float32(scale), dtype)
    return out


def _oracle_rows(restatement, x, dtype, temps, topps, topks, seeds):
    want = np.empty(len(seeds), dtype=np.int64)
    for r in range(len(seeds)):
        t = max(float(temps[r]), 0.0)
        want[r] = restatement.sample_rows(x[r:r + 1], t, float(topps[r]), seeds[r:r + 1], dtype=dtype,
                                          topk=int(topks[r]))[0]
    return want


@pytest.mark.parametrize("dtype", ["bf16", "fp16", "fp32"])
def test_rows_with_their_own_settings(cuda_device, restatement, dtype):
    rng = np.random.default_rng(31)
    rows, vocab = 48, 12000
    v = (-1.2 * np.log(1.0 + rng.permuted(np.tile(np.arange(vocab, dtype=np.float32), (rows, 1)), axis=1))
         + 0.5 * rng.standard_normal((rows, vocab))).astype(np.float32)
    x = _to_storage(v, dtype)
    temps = rng.choice([0.0, 0.3, 0.7, 1.0, -1.0], size=rows).astype(np.float32)  # -1: clamped to greedy
    topps = rng.choice([0.5, 0.9, 0.95, 1.0, 0.0], size=rows).astype(np.float32)
    topks = rng.choice([0, 0, 1, 40, vocab + 5], size=rows).astype(np.int32)
    seeds = rng.integers(1, 2**62, size=rows).astype(np.uint64)
    want = _oracle_rows(restatement, x, dtype, temps, topps, topks, seeds)
    s = Sampler(vocab, 0.8, 0.9, 0, device=cuda_device)
    try:
        t = to_device(x, dtype, cuda_device)
        states = seeds_to_states(seeds, cuda_device)
        ids = s.sample_rows_ex(t, states, temperature=torch.from_numpy(temps).to(cuda_device),
                               topp=torch.from_numpy(topps).to(cuda_device),
                               topk=torch.from_numpy(topks).to(cuda_device))
        torch.cuda.synchronize()
        assert np.array_equal(ids.cpu().numpy(), want)
        # greedy rows draw no coin: their states are untouched; the others advanced once
        after = states.cpu().numpy().view(np.uint64)
        greedy = temps <= 0
        assert np.array_equal(after[greedy], seeds[greedy]) and (after[~greedy] != seeds[~greedy]).all()
        # only some settings per row: the rest is the handle's
        ids2 = s.sample_rows_ex(t, seeds_to_states(seeds, cuda_device),
                                topp=torch.from_numpy(topps).to(cuda_device))
        want2 = _oracle_rows(restatement, x, dtype, np.full(rows, 0.8), topps, np.zeros(rows), seeds)
        assert np.array_equal(ids2.cpu().numpy(), want2)
    finally:
        s.close()


@pytest.mark.parametrize("dtype", ["bf16", "fp32"])
def test_mask_bias_and_multiply_processors_on_device(cuda_device, restatement, dtype):
    rng = np.random.default_rng(32)
    rows, vocab = 12, 9000
    v = (2.0 * rng.standard_normal((rows, vocab))).astype(np.float32)
    x = _to_storage(v, dtype)
    seeds = rng.integers(1, 2**62, size=rows).astype(np.uint64)
    # per-row edit lists: mask the current best token, bias a few others, some ids out of range
    per_row, ids, bias, offsets = [], [], [], [0]
    for r in range(rows):
        best = int(np.argmax(W.to_f32(x[r:r + 1], dtype)[0]))
        edits = [(best, -np.inf), (int(rng.integers(vocab)), 3.5), (int(rng.integers(vocab)), -2.25),
                 (vocab + 7, 1.0), (-3, 1.0)]
        if r % 3 == 0:
            edits = edits[:1]
        per_row.append(edits)
        ids += [e[0] for e in edits]
        bias += [e[1] for e in edits]
        offsets.append(len(ids))
    dev = cuda_device
    t_ids = torch.tensor(ids, dtype=torch.int32, device=dev)
    t_bias = torch.tensor(bias, dtype=torch.float32, device=dev)
    t_off = torch.tensor(offsets, dtype=torch.int64, device=dev)
    for temperature, topp, scale in ((0.0, 0.9, 1.0), (0.8, 0.9, 1.0), (0.8, 0.9, 0.5), (1.0, 1.0, 1.75)):
        xp = _host_process(x, dtype, per_row, scale)
        want = restatement.sample_rows(xp, temperature, topp, seeds, dtype=dtype)
        s = Sampler(vocab, temperature, topp, 0, device=dev)
        try:
            t = to_device(x, dtype, dev)
            got = s.sample_rows_ex(t, seeds_to_states(seeds, dev), scale=scale, edit_ids=t_ids, edit_bias=t_bias,
                                   edit_offsets=t_off).cpu().numpy()
            torch.cuda.synchronize()
            assert np.array_equal(got, want), (temperature, topp, scale)
            # in place, like a processor: the edited logits changed, nothing else did
            back = t.cpu()
            back = back.numpy() if dtype == "fp32" else back.view(torch.int16).numpy().view(np.uint16)
            assert np.array_equal(back.view(np.uint8), _host_process(x, dtype, per_row, 1.0).view(np.uint8))
        finally:
            s.close()
    # one edit list for every row (no offsets): a banned-token list
    shared = [(5, -np.inf), (6, -np.inf), (7, 10.0)]
    xp = _host_process(x, dtype, [shared] * rows, 1.0)
    want = restatement.sample_rows(xp, 0.7, 0.9, seeds, dtype=dtype)
    s = Sampler(vocab, 0.7, 0.9, 0, device=dev)
    try:
        got = s.sample_rows_ex(to_device(x, dtype, dev), seeds_to_states(seeds, dev),
                               edit_ids=torch.tensor([e[0] for e in shared], dtype=torch.int32, device=dev),
                               edit_bias=torch.tensor([e[1] for e in shared], dtype=torch.float32, device=dev))
        assert np.array_equal(got.cpu().numpy(), want)
    finally:
        s.close()


def test_processor_chain_changes_the_argmax_like_the_runner_test(cuda_device):
    """test_text_llm_runner.cpp:656-715: logits {.., 3 best}; masking 3 gives 2; masking 2 too gives 1."""
    logits = torch.tensor([[0.1, 0.2, 0.3, 0.4]], device=cuda_device)
    s = Sampler(4, 0.0, 0.9, 0, device=cuda_device)
    try:
        def run(banned):
            t = logits.clone()
            ids = torch.tensor(banned, dtype=torch.int32, device=cuda_device)
            bias = torch.full((len(banned),), float("-inf"), device=cuda_device)
            return int(s.sample_rows_ex(t, None, edit_ids=ids, edit_bias=bias)[0]) if banned else \
                int(s.sample_rows_ex(t, None)[0])
        assert run([]) == 3 and run([3]) == 2 and run([3, 2]) == 1
        with pytest.raises(SamplerError):
            s.sample_rows_ex(logits.clone(), None, scale=0.0)
        u16 = torch.zeros((1, 4), dtype=torch.uint16, device=cuda_device)
        with pytest.raises(SamplerError):
            s.sample_rows_ex(u16, None)
    finally:
        s.close()
