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
from .model import Model, Poisoned, StepEntry
from .scheduler import Request, Scheduler


@dataclass
class Finished:
    request_id: int
    prompt_tokens: int
    token_ids: List[int]
    finish_reason: str     # "stop" (end-of-sequence id) or "length"


@dataclass
class _InFlight:
    """A step that was launched and whose sampled ids have not been read back yet."""
    sampled_for: List[Request]
    ids: Optional[torch.Tensor]          # int32 on the device, one per request of `sampled_for`
    host: Optional[torch.Tensor]         # pinned: the ids and the status word, once `ready` has happened
    ready: Optional[torch.cuda.Event]
    all_decode: bool                     # every entry was a single decoded token


class Engine:
    """`run_ahead`: when the step after the one in flight can be foreseen (the same requests
    decode again: nothing waits for admission, nobody reaches its token limit), it is launched
    BEFORE the ids of the step in flight are read back, fed on the device by those ids.  The
    host's bookkeeping then runs beside the device's work instead of between two steps.  A
    request that turns out to have met an end-of-sequence id has one row computed in vain;
    its result is dropped.  Tokens, order and finish reasons are the same as without it."""

    def __init__(self, model: Model, max_batch_tokens: int = 256, prefill_chunk: int = 128,
                 policy: str = "mixed", admission_reserve_steps: int = 16, run_ahead: bool = True):
        if model.cache is None:
            raise ValueError("the model has no cache; call allocate_cache first")
        self.model = model
        self.scheduler = Scheduler(model.cache, max_batch_tokens, prefill_chunk, policy, admission_reserve_steps)
        self.sampler = Sampler(model.rt.device, model.status)
        self.eos = set(model.plan.eos_token_ids)
        self.run_ahead = run_ahead
        self._next_id = 0
        self.steps = 0
        self.steps_ahead = 0      # how many of them were launched before the step before was read back
        self.batch_log: List[Dict[str, int]] = []   # per step: prefill and decode tokens (a step trace)
        self._in_flight: Optional[_InFlight] = None
        # Two pinned buffers for the ids coming back (one being read while the next is filled), and two device
        # buffers for the ids and the status word of a step (the ids of the step in flight feed the step launched
        # ahead of it, whose own ids go to the other buffer).
        self._readback = [torch.empty(model.cache.max_requests + 1, dtype=torch.int32).pin_memory() for _ in range(2)]
        self._sampled = [torch.empty(model.cache.max_requests + 1, dtype=torch.int32, device=model.rt.device) for _ in range(2)]
        self._readback_turn = 0

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

    # ---- launching a step
    def _sample_and_send_back(self, logits: torch.Tensor, sampled_for: List[Request], ahead: int, all_decode: bool) -> _InFlight:
        """Samples one id per wanted row and starts their copy to the host.  `ahead` is how
        many tokens of each request are still on their way (1 when launching ahead)."""
        if logits is None or logits.dim() != 2 or logits.shape[0] != len(sampled_for):
            got = "no logits" if logits is None else f"logits of shape {tuple(logits.shape)}"
            self.model._poison(f"the step function returned {got} for {len(sampled_for)} wanted rows")
            raise RuntimeError(f"the step function returned {got} for {len(sampled_for)} wanted rows")
        temps = [r.params.temperature for r in sampled_for]
        uniforms = [uniform_for(r.params.seed, r.request_id, len(r.generated) + ahead) for r in sampled_for]
        n = len(sampled_for)
        packed = self._sampled[self._readback_turn]
        ids = self.sampler.sample(logits, temps, uniforms, out=packed[:n])
        packed[n:n + 1].copy_(self.model.status)
        host = self._readback[self._readback_turn][:n + 1]
        self._readback_turn ^= 1
        host.copy_(packed[:n + 1], non_blocking=True)     # one copy: the tokens and the status word
        ready = torch.cuda.Event()
        ready.record()
        return _InFlight(sampled_for, ids, host, ready, all_decode)

    def _launch(self) -> Optional[_InFlight]:
        """Admits, plans and launches one step from what the host knows."""
        sched = self.scheduler
        sched.admit(self.model.open_request)
        slices = sched.plan()
        if not slices:
            return None
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
        if not sampled_for:
            return _InFlight([], None, None, None, False)
        return self._sample_and_send_back(logits, sampled_for, 0, all(not s.is_prefill for s in slices))

    def _launch_ahead(self, before: _InFlight) -> Optional[_InFlight]:
        """The step after `before`, launched while the ids of `before` are still on the
        device; None if that step cannot be foreseen."""
        sched = self.scheduler
        if not before.all_decode or sched.waiting or len(before.sampled_for) != len(sched.active):
            return None
        for r in before.sampled_for:
            if r.finish_reason or len(r.generated) + 2 > r.params.max_tokens:      # ends with the token in flight
                return None
        # The plan does not look at token values: with every request past its prompt it is
        # the same batch again.
        slices = sched.plan()
        if (len(slices) != len(before.sampled_for) or any(s.is_prefill for s in slices)
                or any(s.request is not r for s, r in zip(slices, before.sampled_for))):
            return None
        entries = [StepEntry(r.slot, [0], [0]) for r in before.sampled_for]
        logits = self.model.step(entries, device_tokens=before.ids)
        self.steps += 1
        self.steps_ahead += 1
        self.batch_log.append({"prefill": 0, "decode": len(entries)})
        return self._sample_and_send_back(logits, before.sampled_for, 1, True)

    # ---- reading a step back
    def _finish(self, step: _InFlight) -> List[Finished]:
        finished: List[Finished] = []
        if not step.sampled_for:
            return finished
        step.ready.synchronize()
        values = step.host.tolist()
        # The whole set of results is checked before any of it is handed out, as the reference
        # does (src/engine.cpp:489-511): a status word a kernel set, or an id that is no token,
        # poisons the model and no request of the step advances.
        if values[-1]:
            self.model.check_status()
        vocab = self.model.plan.vocab_size
        for r, token in zip(step.sampled_for, values[:-1]):
            if not r.finish_reason and not 0 <= token < vocab:
                why = "the logits were not finite" if token < 0 else f"the sampled id {token} is no token"
                self.model._poison(f"request {r.request_id}: {why}")
                raise RuntimeError(f"request {r.request_id}: {why}")
        for r, token in zip(step.sampled_for, values[:-1]):
            if r.finish_reason:
                continue        # it ended with the step before; this row ran ahead in vain
            r.generated.append(token)
            if token in self.eos and not r.params.ignore_eos:
                r.finish_reason = "stop"
            elif len(r.generated) >= r.params.max_tokens:
                r.finish_reason = "length"
            if r.finish_reason:
                self.model.close_request(r.slot)
                self.scheduler.release(r)
                finished.append(Finished(r.request_id, len(r.prompt), list(r.generated), r.finish_reason))
        return finished

    def step(self) -> List[Finished]:
        """One iteration; returns the requests that finished in it.  A poisoned model ends
        generation: the call raises `Poisoned` and no further token is handed out."""
        if self.model.poisoned is not None:
            self._in_flight = None
            raise Poisoned(f"the model is poisoned and must not be used further ({self.model.poisoned})")
        current, self._in_flight = self._in_flight, None
        if current is not None and all(r.finish_reason for r in current.sampled_for):
            current = None      # every request of the step that ran ahead has ended meanwhile
        if current is None:
            current = self._launch()
            if current is None:
                return []
        if self.run_ahead and current.sampled_for:
            self._in_flight = self._launch_ahead(current)
        return self._finish(current)

    def run(self) -> List[Finished]:
        """Runs until every submitted request has finished; results in submission order."""
        done: List[Finished] = []
        while self.has_work():
            done += self.step()
        return sorted(done, key=lambda f: f.request_id)
