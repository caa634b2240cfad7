"""B200-native token sampler: a drop-in for the sampling step of ExecuTorch's LLM runner
(extension/llm/sampler). CUDA only; see include/etb200_sampler.h for the C ABI."""

__all__ = ["Sampler", "sample_from_logits", "sample_all_from_logits", "logits_to_token",
           "seeds_to_states", "ShardedSampler", "shard_rows", "LogitProcessor",
           "apply_logit_processors", "TokenGenerator", "Stats"]


def __getattr__(name):
    if name in ("Sampler", "sample_from_logits", "sample_all_from_logits", "logits_to_token",
                "seeds_to_states", "K_TOPP"):
        from . import sampler
        return getattr(sampler, name)
    if name in ("ShardedSampler", "shard_rows"):
        from . import sharded
        return getattr(sharded, name)
    if name in ("LogitProcessor", "apply_logit_processors", "TokenGenerator", "Stats"):
        from . import generator
        return getattr(generator, name)
    raise AttributeError(name)
