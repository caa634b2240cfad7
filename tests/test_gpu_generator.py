"""The caller side of the sampler on the GPU: logit-processor chain and decode loop, mirrored
from the reference's tests (extension/llm/sampler/test/test_logit_processor.cpp:109-223,
extension/llm/runner/test/test_text_llm_runner.cpp:236-301,656-735)."""
import numpy as np
import pytest
import torch

import json

from executorch_b200 import (LogitProcessor, Sampler, Stats, TokenGenerator, _lib, apply_logit_processors,
                             logits_to_token)

pytestmark = pytest.mark.gpu


class AddBias(LogitProcessor):
    def __init__(self, token, bias):
        self.token, self.bias = token, bias

    def process(self, logits):
        if logits.dtype != torch.float32:
            return _lib.INVALID_ARGUMENT  # processors declare their own dtype expectations
        self.last_position(logits)[:, self.token] += self.bias
        return _lib.OK


class Multiply(LogitProcessor):
    def __init__(self, factor):
        self.factor = factor

    def process(self, logits):
        self.last_position(logits).mul_(self.factor)
        return _lib.OK


class MaskToken(LogitProcessor):
    def __init__(self, token):
        self.token = token

    def process(self, logits):
        v = self.last_position(logits)
        if 0 <= self.token < v.shape[-1]:  # out-of-range ids are a no-op
            v[:, self.token] = float("-inf")
        return _lib.OK


def test_single_processor_mutates_in_place(cuda_device):
    t = torch.tensor([[0.1, 0.2, 0.3, 0.4]], device=cuda_device)
    assert AddBias(1, 10.0).process(t) == _lib.OK
    assert torch.allclose(t.cpu(), torch.tensor([[0.1, 10.2, 0.3, 0.4]]))


def test_chain_runs_in_registration_order(cuda_device):
    t = torch.tensor([[1.0, 2.0, 3.0, 4.0]], device=cuda_device)
    assert apply_logit_processors([AddBias(0, 1.0), Multiply(2.0)], t) == _lib.OK
    assert torch.allclose(t.cpu(), torch.tensor([[4.0, 4.0, 6.0, 8.0]]))  # (1+1)*2, not 1*2+1


def test_mask_changes_the_sampled_token_and_out_of_range_is_a_noop(cuda_device):
    t = torch.tensor([[0.1, 0.2, 0.3, 0.4]], device=cuda_device)
    assert logits_to_token(t, 0.0) == 3
    MaskToken(3).process(t)
    assert logits_to_token(t, 0.0) == 2
    MaskToken(2).process(t)
    assert logits_to_token(t, 0.0) == 1
    before = t.clone()
    MaskToken(99).process(t)
    MaskToken(-1).process(t)
    assert torch.equal(t, before)
    # a masked token is never drawn, whatever the coin
    s = Sampler(4, 1.0, 0.9, 1, device=cuda_device)
    assert {s.sample(t[0]) for _ in range(200)} <= {0, 1}
    s.close()


def test_rank3_touches_the_last_position_only_and_dtype_is_checked(cuda_device):
    t = torch.zeros((1, 3, 4), device=cuda_device)
    assert AddBias(2, 5.0).process(t) == _lib.OK
    assert float(t[0, 2, 2]) == 5.0 and float(t[0, :2].abs().sum()) == 0.0
    assert AddBias(0, 1.0).process(t.to(torch.float16)) == _lib.INVALID_ARGUMENT
    assert apply_logit_processors([AddBias(0, 1.0), Multiply(3.0)], t.to(torch.float16)) == _lib.INVALID_ARGUMENT


class FakeModel:
    """Stands in for TextDecoderRunner::step: returns a fixed [1, V] logits tensor."""

    def __init__(self, logits):
        self.logits, self.calls = logits, 0

    def __call__(self, tokens, pos):
        self.calls += 1
        return self.logits.clone()


def test_generate_calls_back_once_per_token_and_counts_steps(cuda_device):
    model = FakeModel(torch.tensor([[0.1, 0.2, 0.3, 0.4]], device=cuda_device))
    s = Sampler(4, 0.0, 0.9, 0, device=cuda_device)
    g = TokenGenerator(model, s, eos_ids={100})
    seen = []
    n = g.generate([1, 2, 3], start_pos=3, max_new_tokens=10, temperature=0.0, token_callback=seen.append)
    assert n == 10 and len(seen) == 10 and model.calls == 10 and set(seen) == {"3"}
    s.close()


def test_generate_fills_the_reference_stats_and_report_line(cuda_device):
    """The counters a decode loop feeds in the reference's Stats (stats.h:24-75) and the
    JSON keys of its PyTorchObserver line (stats.h:113-165)."""
    model = FakeModel(torch.tensor([[0.1, 0.2, 0.3, 0.4]], device=cuda_device))
    s = Sampler(4, 0.5, 0.9, 3, device=cuda_device)
    st = Stats()
    g = TokenGenerator(model, s, stats=st)
    n = g.generate([5, 6], start_pos=2, max_new_tokens=7, temperature=0.5)
    assert n == 7 and st.num_generated_tokens == 7 and st.num_prompt_tokens == 2
    assert st.aggregate_sampling_time_ms > 0 and g.sampling_time_ms == st.aggregate_sampling_time_ms
    assert st.aggregate_model_execution_time_ms > 0
    assert 0 < st.inference_start_ms <= st.first_token_ms <= st.inference_end_ms
    line = st.report_line()
    assert line.startswith("PyTorchObserver {")
    d = json.loads(line[len("PyTorchObserver "):])
    keys = list(d)
    assert keys[-1] == "SCALING_FACTOR_UNITS_PER_SECOND" and d[keys[-1]] == 1000
    for k in ("prompt_tokens", "generated_tokens", "model_load_start_ms", "model_load_end_ms",
              "inference_start_ms", "inference_end_ms", "model_execution_start_ms",
              "model_execution_end_ms", "prompt_eval_end_ms", "first_token_ms",
              "aggregate_sampling_time_ms", "aggregate_model_execution_time_ms"):
        assert k in d
    assert d["generated_tokens"] == 7
    st.reset()
    assert st.num_generated_tokens == 0 and st.aggregate_sampling_time_ms == 0
    s.close()


def test_generate_with_processors_changes_argmax(cuda_device):
    model = FakeModel(torch.tensor([[0.1, 0.2, 0.3, 0.4]], device=cuda_device))
    s = Sampler(4, 0.0, 0.9, 0, device=cuda_device)
    g = TokenGenerator(model, s)
    out = []
    g.generate([1], 1, 1, 0.0, out.append)
    g.add_logit_processor(MaskToken(3))
    g.generate([1], 1, 1, 0.0, out.append)
    g.add_logit_processor(MaskToken(2))
    g.generate([1], 1, 1, 0.0, out.append)
    assert out == ["3", "2", "1"]
    s.close()


def test_generate_rejects_temperature_outside_unit_interval_before_stepping(cuda_device):
    model = FakeModel(torch.tensor([[0.1, 0.2, 0.3, 0.4]], device=cuda_device))
    s = Sampler(4, 0.0, 0.9, 0, device=cuda_device)
    g = TokenGenerator(model, s)
    for bad in (-0.1, 1.5):
        with pytest.raises(_lib.SamplerError) as e:
            g.generate([1], 1, 5, bad)
        assert e.value.code == _lib.INVALID_ARGUMENT
    assert model.calls == 0
    s.close()


def test_generate_stops_on_eos_and_on_stop(cuda_device, restatement):
    logits = torch.tensor([[0.0, 5.0, 0.0, 0.0]], device=cuda_device)
    s = Sampler(4, 0.0, 0.9, 0, device=cuda_device)
    g = TokenGenerator(FakeModel(logits), s, eos_ids={1})
    assert g.generate([0], 0, 10, 0.0) == 1  # the first sampled token is EOS
    g2 = TokenGenerator(FakeModel(logits), s, eos_ids={1}, ignore_eos=True)
    assert g2.generate([0], 0, 4, 0.0) == 4
    g3 = TokenGenerator(FakeModel(torch.zeros((1, 4), device=cuda_device)), s)
    g3.generate([0], 0, 10, 0.0, token_callback=lambda _: g3.stop())
    s.close()
    # sampled decode loop with temperature: the sampler state evolves exactly like the
    # reference's single Sampler owned by the decoder runner
    x = np.random.default_rng(4).standard_normal((1, 5000)).astype(np.float32) * 2
    model = FakeModel(torch.from_numpy(x).to(cuda_device))
    s = Sampler(5000, 0.3, 0.9, 2024, device=cuda_device)
    toks = []
    TokenGenerator(model, s, decode=lambda p, c: str(c)).generate([7], 0, 40, 0.9, toks.append)
    want = restatement.sample_sequence(x[0], 0.9, 0.9, 2024, 40)
    assert [int(t) for t in toks] == list(want)
    s.close()
