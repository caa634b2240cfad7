"""Host-side callers of the sampler, mirrored from the reference's LLM runner so that the
sampling path can be driven the way the reference drives it:

* ``LogitProcessor`` / ``apply_logit_processors`` -- the in-place pre-sampling hooks of
  extension/llm/sampler/logit_processor.h:34-40, run in registration order as in
  extension/llm/runner/text_token_generator.h:143. Processors receive the DEVICE logits
  tensor and edit it in place (rank 2: the whole last dimension; rank 3: the last sequence
  position only).
* ``TokenGenerator`` -- the decode loop of TextTokenGenerator::generate
  (text_token_generator.h:83-186): step the model, run the processors, sample one token,
  report it, stop on EOS / stop() / max_new_tokens. The model forward is any callable
  ``step(tokens, pos) -> logits tensor on the GPU`` (the reference's TextDecoderRunner::step,
  text_decoder_runner.h:41); tokenizer decoding is any callable ``decode(prev, cur) -> str``.

* ``Stats`` -- the counters of extension/llm/runner/stats.h that the decode loop feeds
  (sampling and model-execution time, token counts, first-token and end timestamps), with the
  reference's JSON keys and its ``PyTorchObserver`` report line (stats.h:113-173).

This is orchestration only; all arithmetic happens in the CUDA library.
"""
from __future__ import annotations

import json
import threading
import time
from typing import Callable, Iterable, Sequence

import torch

from . import _lib
from .sampler import Sampler, sample_from_logits


class LogitProcessor:
    """In-place logit transform applied between the model forward pass and the sampler.
    ``process`` returns an error code (``_lib.OK`` = 0 to continue, anything else aborts the
    chain), like ``Error LogitProcessor::process(Tensor)``."""

    def process(self, logits: torch.Tensor) -> int:  # pragma: no cover - interface
        raise NotImplementedError

    @staticmethod
    def last_position(logits: torch.Tensor) -> torch.Tensor:
        """View of what a processor may touch: [batch, vocab] of a rank-2 tensor, or the last
        sequence position of a rank-3 [batch, seq, vocab] tensor."""
        if logits.dim() == 3:
            return logits[:, logits.shape[1] - 1, :]
        return logits


def apply_logit_processors(processors: Iterable[LogitProcessor], logits: torch.Tensor) -> int:
    """Runs the processors in order; each sees the edits of the ones before it. Stops at the
    first non-Ok code and returns it (text_token_generator.h:143, :236-244)."""
    for p in processors:
        code = p.process(logits)
        if code != _lib.OK:
            return code
    return _lib.OK


class Stats:
    """The fields of the reference's ``Stats`` (stats.h:24-75) that a decode loop can fill,
    in the reference's unit (milliseconds; ``SCALING_FACTOR_UNITS_PER_SECOND`` = 1000).
    Sampling time is device time between CUDA events around the sampling call; model
    execution time is host wall time around ``step`` including its synchronisation by the
    first consumer. Timestamps are host milliseconds since the epoch, like ``time_in_ms``."""

    SCALING_FACTOR_UNITS_PER_SECOND = 1000

    def __init__(self):
        self.reset(all_stats=True)

    def reset(self, all_stats: bool = False) -> None:
        if all_stats:
            self.model_load_start_ms = 0
            self.model_load_end_ms = 0
        self.inference_start_ms = 0
        self.model_execution_start_ms = 0
        self.model_execution_end_ms = 0
        self.prompt_eval_end_ms = 0
        self.first_token_ms = 0
        self.inference_end_ms = 0
        self.aggregate_sampling_time_ms = 0.0
        self.aggregate_model_execution_time_ms = 0.0
        self.num_prompt_tokens = 0
        self.num_generated_tokens = 0

    @staticmethod
    def time_in_ms() -> int:
        return int(time.time() * 1000)

    def to_json(self) -> str:
        """Same keys, in the same order, as ``stats_to_json_string`` (stats.h:113-161); the
        optional GPU memory fields are left out, as the reference does when they are unset."""
        d = {}
        prefill_ms = self.prompt_eval_end_ms - self.inference_start_ms
        if prefill_ms > 0:
            d["prefill_token_per_sec"] = self.num_prompt_tokens / prefill_ms * self.SCALING_FACTOR_UNITS_PER_SECOND
        decode_ms = self.inference_end_ms - self.prompt_eval_end_ms
        if decode_ms > 0:
            d["decode_token_per_sec"] = self.num_generated_tokens / decode_ms * self.SCALING_FACTOR_UNITS_PER_SECOND
        d["prompt_tokens"] = self.num_prompt_tokens
        d["generated_tokens"] = self.num_generated_tokens
        for k in ("model_load_start_ms", "model_load_end_ms", "inference_start_ms", "inference_end_ms",
                  "model_execution_start_ms", "model_execution_end_ms", "prompt_eval_end_ms", "first_token_ms",
                  "aggregate_sampling_time_ms", "aggregate_model_execution_time_ms"):
            d[k] = getattr(self, k)
        d["SCALING_FACTOR_UNITS_PER_SECOND"] = self.SCALING_FACTOR_UNITS_PER_SECOND
        return json.dumps(d, separators=(",", ":"))

    def report_line(self) -> str:
        """The line ``print_report`` emits for dashboards (stats.h:164-165)."""
        return "PyTorchObserver " + self.to_json()


class TokenGenerator:
    """``generate(tokens, start_pos, max_new_tokens, temperature, token_callback)`` as
    TextTokenGenerator::generate. ``sampler`` plays the role of the Sampler that
    TextDecoderRunner owns (text_decoder_runner.h:84-94,107): its temperature is set per
    call with ``set_temperature`` and its RNG state evolves across steps."""

    def __init__(self, step: Callable[[Sequence[int], int], torch.Tensor], sampler: Sampler,
                 eos_ids: Iterable[int] = (), decode: Callable[[int, int], str] | None = None,
                 use_kv_cache: bool = True, ignore_eos: bool = False, stats: Stats | None = None):
        self.step = step
        self.sampler = sampler
        self.eos_ids = set(eos_ids)
        self.decode = decode or (lambda prev, cur: str(cur))
        self.use_kv_cache = use_kv_cache
        self.ignore_eos = ignore_eos
        self.processors: list[LogitProcessor] = []
        self._should_stop = threading.Event()
        self.stats = stats if stats is not None else Stats()

    @property
    def sampling_time_ms(self) -> float:
        """``aggregate_sampling_time_ms`` of the attached Stats."""
        return self.stats.aggregate_sampling_time_ms

    def add_logit_processor(self, p: LogitProcessor) -> None:
        self.processors.append(p)

    def stop(self) -> None:
        self._should_stop.set()

    def generate(self, tokens: Sequence[int], start_pos: int, max_new_tokens: int,
                 temperature: float = 0.0,
                 token_callback: Callable[[str], None] | None = None) -> int:
        if len(tokens) == 0:
            raise ValueError("Token generation loop shouldn't take empty tokens")
        if not (0.0 <= temperature <= 1.0):
            # checked before the model is ever stepped (text_token_generator.h:91-95)
            raise _lib.SamplerError(_lib.INVALID_ARGUMENT, f"Temperature must be in [0, 1], got {temperature}")
        pos = start_pos
        cur = int(tokens[-1])
        history = [cur] if self.use_kv_cache else [int(t) for t in tokens]
        self._should_stop.clear()
        self.sampler.set_temperature(temperature)
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        st = self.stats
        if st.inference_start_ms == 0:
            st.inference_start_ms = st.time_in_ms()
        if st.prompt_eval_end_ms == 0:
            st.prompt_eval_end_ms = st.inference_start_ms  # the prompt was evaluated by the caller
            st.num_prompt_tokens = len(tokens)
        while pos < start_pos + max_new_tokens:
            st.model_execution_start_ms = st.time_in_ms()
            m0 = time.perf_counter()
            logits = self.step(history, pos)
            st.aggregate_model_execution_time_ms += (time.perf_counter() - m0) * 1e3
            st.model_execution_end_ms = st.time_in_ms()
            prev = cur
            code = apply_logit_processors(self.processors, logits)
            if code != _lib.OK:
                raise _lib.SamplerError(code, "a logit processor aborted the chain")
            t0.record()
            cur = sample_from_logits(logits, self.sampler)
            t1.record()
            t1.synchronize()
            st.aggregate_sampling_time_ms += t0.elapsed_time(t1)
            st.num_generated_tokens += 1
            if st.first_token_ms == 0:
                st.first_token_ms = st.time_in_ms()
            pos += 1
            if self.use_kv_cache:
                history[0] = cur
            else:
                history.append(cur)
            if token_callback is not None:
                token_callback(self.decode(prev, cur))
            if self._should_stop.is_set():
                break
            if not self.ignore_eos and cur in self.eos_ids:
                break
        st.inference_end_ms = st.time_in_ms()
        return pos - start_pos
