"""The Python entry point.

    llm = LLM(model_dir, dtype="bfloat16")
    results = llm.generate([[1, 2, 3], [4, 5]], max_tokens=16, temperature=0.7, seed=7)

Token ids in, token ids out; text is not this engine's business (the reference's
tokenizer is llama.cpp's, src/minillm/tokenizer.cpp).
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Union

from ..sampling.sampler import SamplingParams
from .engine import Engine, Finished
from .loading import load_model
from .model import CacheConfig, Model


class LLM:
    def __init__(self, model: Union[str, Model], dtype: str = "bfloat16", max_model_len: int = 0,
                 max_requests: int = 8, page_size: int = 16, num_pages: int = 0,
                 max_batch_tokens: int = 4096, prefill_chunk: int = 2048, policy: str = "mixed",
                 device: str = "cuda:0", run_ahead: bool = True):
        """`model`: a folder with config.json and model.safetensors, or a built Model.
        `num_pages` 0 sizes the pool for `max_requests` requests of `max_model_len`.
        `run_ahead`: launch a foreseeable decode step before the last one is read back.
        `max_batch_tokens`, `prefill_chunk`: the reference's names (EngineConfig, its
        defaults 256 and 128 fit a 0.6B model); the defaults here are sized for a B200, where
        a product of fewer than some hundred rows is bound by reading the weights, so a
        larger prompt portion costs a step little.  Both are capped by the model length."""
        if isinstance(model, Model):
            self.model = model
            if model.cache is None:
                raise ValueError("a Model passed to LLM must have its cache allocated")
        else:
            self.model = load_model(model, dtype, None, device)
            max_len = max_model_len or self.model.plan.max_positions
            pages = num_pages or max_requests * ((max_len + page_size - 1) // page_size)
            self.model.allocate_cache(CacheConfig(page_size=page_size, num_pages=pages, max_requests=max_requests,
                                                  max_model_len=max_len))
        limit = self.model.cache_config.max_model_len
        prefill_chunk = max(1, min(prefill_chunk, limit))
        max_batch_tokens = max(self.model.cache.max_requests, prefill_chunk, min(max_batch_tokens, limit * self.model.cache.max_requests))
        self.engine = Engine(self.model, max_batch_tokens, prefill_chunk, policy, run_ahead=run_ahead)

    def generate(self, prompts: Sequence[Sequence[int]], max_tokens: int = 32, temperature: float = 0.0,
                 seed: int = 0, ignore_eos: bool = False,
                 params: Optional[Sequence[SamplingParams]] = None) -> List[Finished]:
        """Generates for every prompt (a list of token ids); results come in the order
        of the prompts.  `params` gives each prompt its own sampling parameters."""
        if params is not None and len(params) != len(prompts):
            raise ValueError("one SamplingParams per prompt")
        ids = []
        for i, prompt in enumerate(prompts):
            p = params[i] if params is not None else SamplingParams(max_tokens, temperature, seed, ignore_eos)
            ids.append(self.engine.submit(prompt, p))
        by_id = {f.request_id: f for f in self.engine.run()}
        return [by_id[i] for i in ids]
