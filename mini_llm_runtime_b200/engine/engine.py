"""Generation: requests in, token ids out, through the one step function.

An iteration is the reference's `Engine::iteration` (src/engine.cpp:392-580)
without its server: admit what fits, plan the batch, expand the plan into step
entries (a prompt portion asks for logits only at the prompt's last token; a
decoding request brings its last token), run `Model.step`, sample one token per
wanted row on the device, read the ids back, advance every request, and finish and
free those that hit an end-of-sequence id or their token limit.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import torch

from ..sampling.sampler import Sampler, SamplingParams, uniform_for
from .model import Model, StepEntry
from .scheduler import Request, Scheduler


@dataclass
class Finished:
    request_id: int
    prompt_tokens: int
    token_ids: List[int]
    finish_reason: str     # "stop" (end-of-sequence id) or "length"


class Engine:
    def __init__(self, model: Model, max_batch_tokens: int = 256, prefill_chunk: int = 128,
                 policy: str = "mixed", admission_reserve_steps: int = 16):
        if model.cache is None:
            raise ValueError("the model has no cache; call allocate_cache first")
        self.model = model
        self.scheduler = Scheduler(model.cache, max_batch_tokens, prefill_chunk, policy, admission_reserve_steps)
        self.sampler = Sampler(model.rt.device, model.status)
        self.eos = set(model.plan.eos_token_ids)
        self._next_id = 0
        self.steps = 0
        self.batch_log: List[Dict[str, int]] = []   # per step: prefill and decode tokens (a step trace)

    def submit(self, prompt: Sequence[int], params: Optional[SamplingParams] = None) -> int:
        params = params or SamplingParams()
        vocab = self.model.plan.vocab_size
        prompt = [int(t) for t in prompt]
        if any(t < 0 or t >= vocab for t in prompt):
            raise ValueError(f"a prompt token is outside the vocabulary of {vocab}")
        request = Request(self._next_id, prompt, params)
        self.scheduler.submit(request)
        self._next_id += 1
        return request.request_id

    def has_work(self) -> bool:
        return bool(self.scheduler.waiting or self.scheduler.active)

    def step(self) -> List[Finished]:
        """One iteration; returns the requests that finished in it."""
        sched = self.scheduler
        sched.admit(self.model.open_request)
        slices = sched.plan()
        if not slices:
            return []
        entries, sampled_for = [], []
        for s in slices:
            r = s.request
            if s.is_prefill:
                tokens = r.prompt[r.processed:r.processed + s.tokens]
                last = r.processed + s.tokens == len(r.prompt)
                entries.append(StepEntry(r.slot, tokens, [s.tokens - 1] if last else []))
                if last:
                    sampled_for.append(r)
            else:
                entries.append(StepEntry(r.slot, [r.generated[-1]], [0]))
                sampled_for.append(r)
        logits = self.model.step(entries)
        self.steps += 1
        self.batch_log.append({"prefill": sum(s.tokens for s in slices if s.is_prefill),
                               "decode": sum(1 for s in slices if not s.is_prefill)})
        for s in slices:
            if s.is_prefill:
                s.request.processed += s.tokens
        finished: List[Finished] = []
        if sampled_for:
            temps = [r.params.temperature for r in sampled_for]
            uniforms = [uniform_for(r.params.seed, r.request_id, len(r.generated)) for r in sampled_for]
            ids = self.sampler.sample(logits, temps, uniforms)
            both = torch.cat([ids, self.model.status]).cpu()      # one read: the tokens and the status word
            if int(both[-1]):
                self.model.check_status()
            for r, token in zip(sampled_for, both[:-1].tolist()):
                if token < 0:
                    raise RuntimeError(f"request {r.request_id}: the logits were not finite")
                r.generated.append(token)
                if token in self.eos and not r.params.ignore_eos:
                    r.finish_reason = "stop"
                elif len(r.generated) >= r.params.max_tokens:
                    r.finish_reason = "length"
                if r.finish_reason:
                    self.model.close_request(r.slot)
                    sched.release(r)
                    finished.append(Finished(r.request_id, len(r.prompt), list(r.generated), r.finish_reason))
        return finished

    def run(self) -> List[Finished]:
        """Runs until every submitted request has finished; results in submission order."""
        done: List[Finished] = []
        while self.has_work():
            done += self.step()
        return sorted(done, key=lambda f: f.request_id)
