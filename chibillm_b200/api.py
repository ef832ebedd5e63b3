"""The Python entry point: load a model folder, generate from token ids."""
from __future__ import annotations

from typing import List, Optional, Sequence

from .engine.engine import InferenceEngine
from .engine.runner import ModelRunner
from .engine.scheduler import SchedulerConfig
from .sampling.sampler import SamplingParams

KV_PAGE_SIZE = 16   # tokens per cache page, the reference's block size (src/cli_options.h:15)


class LLM:
    """A loaded model with its cache and scheduler.

    ``context_length`` is the most tokens (prompt plus output) of one request;
    ``kv_cache_tokens`` the size of the shared cache pool (default: enough for
    ``max_sequences`` requests of ``context_length``).  The option names are the
    reference's command-line flags (src/cli_options.cc:13-25).  The defaults of
    the scheduler are sized for a B200 (64 requests, steps of 4,096 tokens, prompt
    portions of 1,024 while others wait or decode); the reference's own, sized for
    a laptop GPU, are 4 requests, 128 tokens and 64 (src/scheduler.h:30-39)."""

    def __init__(self, model_dir: Optional[str], dtype: str = "bfloat16", device: str = "cuda:0",
                 context_length: int = 4096, kv_cache_tokens: Optional[int] = None,
                 max_sequences: int = 64, max_batch_tokens: int = 4096, prefill_chunk_tokens: int = 1024,
                 page_size: int = KV_PAGE_SIZE, kernels=None, random_config: Optional[dict] = None,
                 random_seed: int = 0):
        if context_length <= 0 or context_length % page_size != 0:
            raise ValueError(f"context_length must be a positive multiple of {page_size}")
        pool = kv_cache_tokens if kv_cache_tokens is not None else context_length * max_sequences
        if pool <= 0 or pool % page_size != 0:
            raise ValueError(f"kv_cache_tokens must be a positive multiple of {page_size}")
        if (model_dir is None) == (random_config is None):
            raise ValueError("give a model folder or a configuration for random weights")
        if model_dir is not None:
            self.runner = ModelRunner.from_folder(model_dir, dtype=dtype, device=device,
                                                  page_size=page_size, pool_tokens=pool,
                                                  max_requests=max_sequences, kernels=kernels)
        else:
            self.runner = ModelRunner.from_random(random_config, seed=random_seed, dtype=dtype,
                                                  device=device, page_size=page_size, pool_tokens=pool,
                                                  max_requests=max_sequences, kernels=kernels)
        self.context_length = min(context_length, self.runner.max_context_tokens)
        self.engine = InferenceEngine(self.runner, SchedulerConfig(
            max_sequences=max_sequences, max_batch_tokens=max_batch_tokens,
            prefill_chunk_tokens=prefill_chunk_tokens))

    def generate(self, prompts: Sequence[Sequence[int]], max_tokens: int = 64, temperature: float = 0.0,
                 seed: int = 0, ignore_eos: bool = False) -> List[List[int]]:
        """Generated token ids for each prompt of token ids."""
        params = []
        for p in prompts:
            room = self.context_length - len(p)
            if room < 1:
                raise ValueError(f"a prompt of {len(p)} tokens does not fit a context of {self.context_length}")
            params.append(SamplingParams(max_new_tokens=min(max_tokens, room), ignore_eos=ignore_eos,
                                         temperature=temperature, seed=seed))
        return self.engine.generate(prompts, params)


def generate(model_dir: str, prompts: Sequence[Sequence[int]], max_tokens: int = 64,
             temperature: float = 0.0, seed: int = 0, dtype: str = "bfloat16", **kw) -> List[List[int]]:
    """One call: load ``model_dir`` and generate."""
    return LLM(model_dir, dtype=dtype, **kw).generate(prompts, max_tokens=max_tokens,
                                                      temperature=temperature, seed=seed)
