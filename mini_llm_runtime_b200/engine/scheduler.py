"""Admission and batch planning above the step function.

Policy, restated from the reference (src/engine.cpp:295-355 admission,
src/scheduler.cpp:11-49 planning):

* A request is admitted when a request slot is free and, in every cache group, the
  pages it can ever hold at once fit into the group's unreserved pages.  That worst
  case (`prompt + max_tokens` tokens; for a window group the window plus one step) is
  reserved as credits until the request ends, so an admitted request can never find
  the pool empty: running out of pages shows up as WAITING, never as a failed step.
* A waiting request that does not fit lets younger ones pass until it has waited
  `admission_reserve_steps` planning rounds; from then on it blocks the queue until
  it fits (the reference does this by age in milliseconds).
* A request whose worst case exceeds a whole pool, or that is longer than the model
  allows, is refused at submission.
* If nothing is active and the head of the queue still does not fit, the engine
  raises: no request could ever make progress.
* Planning: under `max_batch_tokens`, every decoding request gets one token first
  (policy "mixed"), then prompts get portions of at most `prefill_chunk` in arrival
  order.  The planner is native code (`csrc/host/scheduler.cpp`).

There is no preemption, swapping or recomputation, as in the reference
(docs/ARCHITECTURE.md:70).
"""
from __future__ import annotations

import ctypes
from collections import deque
from dataclasses import dataclass, field
from typing import Deque, List, Optional, Sequence, Tuple

from ..cache.manager import CacheManager
from ..csrc import build
from ..sampling.sampler import SamplingParams

POLICIES = {"mixed": 0, "prefill_first": 1}


class AdmissionError(ValueError):
    """A request that this engine can never run."""


@dataclass
class Request:
    request_id: int
    prompt: List[int]
    params: SamplingParams
    order: int = 0
    slot: int = -1
    processed: int = 0                     # prompt tokens already in the cache
    generated: List[int] = field(default_factory=list)
    credits: List[int] = field(default_factory=list)   # pages reserved per group
    waited: int = 0
    finish_reason: Optional[str] = None

    @property
    def prefill_remaining(self) -> int:
        return len(self.prompt) - self.processed


@dataclass
class Slice:
    request: Request
    tokens: int
    is_prefill: bool


def _planner():
    lib = build.load("host")
    if not getattr(lib, "_mlr_sched_bound", False):
        i = ctypes.c_int
        p64, p32 = ctypes.POINTER(ctypes.c_int64), ctypes.POINTER(ctypes.c_int32)
        lib.mlr_schedule_batch.argtypes = [i, p64, p32, p64, i, i, i, p64, p32, p32, p32]
        lib.mlr_schedule_batch.restype = i
        lib._mlr_sched_bound = True
    return lib


def schedule_batch(items: Sequence[Tuple[int, int, int]], batch_tokens: int, prefill_chunk: int,
                   policy: str = "mixed") -> List[Tuple[int, int, bool]]:
    """items: (key, prefill_remaining, arrival order).  Returns (key, tokens, is_prefill)
    slices: decodes first, then prompt portions."""
    if policy not in POLICIES:
        raise ValueError(f"policy must be one of {sorted(POLICIES)}")
    n = len(items)
    keys = (ctypes.c_int64 * n)(*[k for k, _, _ in items])
    remaining = (ctypes.c_int32 * n)(*[r for _, r, _ in items])
    order = (ctypes.c_int64 * n)(*[o for _, _, o in items])
    out_keys, out_tokens, out_prefill = (ctypes.c_int64 * n)(), (ctypes.c_int32 * n)(), (ctypes.c_int32 * n)()
    totals = (ctypes.c_int32 * 2)()
    count = _planner().mlr_schedule_batch(n, keys, remaining, order, batch_tokens, prefill_chunk,
                                          POLICIES[policy], out_keys, out_tokens, out_prefill, totals)
    if count < 0:
        raise ValueError("the planner refused its arguments (budget and chunk must be positive)")
    return [(out_keys[i], out_tokens[i], bool(out_prefill[i])) for i in range(count)]


class Scheduler:
    def __init__(self, cache: CacheManager, max_batch_tokens: int = 256, prefill_chunk: int = 128,
                 policy: str = "mixed", admission_reserve_steps: int = 16):
        # Limits as the reference validates them (src/config.cpp:8-36).
        if max_batch_tokens < cache.max_requests:
            raise ValueError(f"max_batch_tokens {max_batch_tokens} must be at least the number of request slots "
                             f"{cache.max_requests}, so that every decoding request fits one step")
        if not 1 <= prefill_chunk <= max_batch_tokens:
            raise ValueError("prefill_chunk must be in [1, max_batch_tokens]")
        if policy not in POLICIES:
            raise ValueError(f"policy must be one of {sorted(POLICIES)}")
        self.cache = cache
        self.max_batch_tokens, self.prefill_chunk, self.policy = max_batch_tokens, prefill_chunk, policy
        self.admission_reserve_steps = admission_reserve_steps
        self.waiting: Deque[Request] = deque()
        self.active: List[Request] = []
        self.reserved = [0] * len(cache.groups)
        self._order = 0

    # ---- admission
    def worst_case_pages(self, total_tokens: int) -> List[int]:
        step = min(self.prefill_chunk, self.max_batch_tokens)
        return [self.cache.peak_pages(g, total_tokens, step) for g in range(len(self.cache.groups))]

    def submit(self, request: Request) -> None:
        request.params.validate()
        total = len(request.prompt) + request.params.max_tokens
        if not request.prompt:
            raise AdmissionError("the prompt is empty")
        if total > self.cache.max_model_len:
            raise AdmissionError(f"prompt ({len(request.prompt)}) plus max_tokens ({request.params.max_tokens}) "
                                 f"exceeds the maximum length {self.cache.max_model_len}")
        need = self.worst_case_pages(total)
        for g, (n, spec) in enumerate(zip(need, self.cache.groups)):
            if n > spec.num_pages:
                raise AdmissionError(f"the request can need {n} pages in cache group {g}, the pool has {spec.num_pages}")
        request.order = self._order
        self._order += 1
        self.waiting.append(request)

    def _fits(self, need: List[int]) -> bool:
        return all(self.reserved[g] + n <= spec.num_pages for g, (n, spec) in enumerate(zip(need, self.cache.groups)))

    def admit(self, open_request) -> List[Request]:
        """Moves waiting requests that fit into the active set; `open_request()` takes
        the slot.  Returns the newly admitted ones."""
        admitted = []
        kept: Deque[Request] = deque()
        blocked = False
        while self.waiting:
            request = self.waiting.popleft()
            need = self.worst_case_pages(len(request.prompt) + request.params.max_tokens)
            if not blocked and self.cache.free_slots() > 0 and self._fits(need):
                request.slot = open_request()
                request.credits = need
                for g, n in enumerate(need):
                    self.reserved[g] += n
                self.active.append(request)
                admitted.append(request)
            else:
                request.waited += 1
                if request.waited > self.admission_reserve_steps:
                    blocked = True
                kept.append(request)
        self.waiting = kept
        if not self.active and self.waiting:
            raise RuntimeError("no request fits an otherwise idle cache pool")
        return admitted

    def release(self, request: Request) -> None:
        for g, n in enumerate(request.credits):
            self.reserved[g] -= n
        request.credits = []
        self.active.remove(request)

    # ---- planning
    def plan(self) -> List[Slice]:
        by_key = {r.request_id: r for r in self.active}
        items = [(r.request_id, r.prefill_remaining, r.order) for r in self.active]
        return [Slice(by_key[k], n, p)
                for k, n, p in schedule_batch(items, self.max_batch_tokens, self.prefill_chunk, self.policy)]
