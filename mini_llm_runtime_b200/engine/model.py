"""The generic model: parts built from a plan, a cache, and ONE step function.

`Model.step(entries)` is the only way tokens reach the kernels.  Generation
(`engine/engine.py`), the command line and trace replay (`bin/trace_run`) all call
it; it is the counterpart of the reference's `CudaRuntime::forward`
(src/minillm/cuda/runtime.cpp:146-254): validate the batch, take cache pages before
any device work, upload the step's metadata in one copy, gather the embeddings, run
the layers in the plan's order, norm and project only the rows whose logits are
wanted, and publish lengths and page maps once the work is enqueued.

A batch is a list of entries, one per request: its next tokens (a portion of its
prompt, or one decoded token) and the places among them whose logits are wanted.
All entries run as one batch of rows; the rows of one request are consecutive
positions that continue what the cache holds for it.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from .. import parts as _builtin_parts  # noqa: F401  (registers the built-in parts)
from ..cache.manager import CacheManager, GroupSpec, OutOfPages
from ..config.base import ModelPlan, PartSpec
from ..config.registry import part_class
from ..csrc import build
from ..parts.base import Block, CacheNeed, RunContext, Segment, StateNeed, StepContext
from ..weights.loader import WeightSpec, merge_specs
from .executor import (NativeStepper, STEP_FAILED, STEP_NO_PAGES, STEP_OK, STEP_POISONED, STEP_REFUSED)
from .runtime import Runtime
from .structure import build_part, build_parts


class StepError(ValueError):
    """A batch the step function refuses; nothing was run and nothing changed."""


class DeviceFault(RuntimeError):
    """A kernel reported a bad index, a bad page or a non-finite value."""


class Poisoned(RuntimeError):
    """The model failed after device work of a step had begun, or a kernel reported a fault:
    what the device holds can no longer be trusted, and the model refuses every further step
    and request (the reference's `poisoned` state: src/minillm/cuda/runtime.cpp:241-253,
    src/minillm/cuda/batch_state.h:9).  Build a new model."""


@dataclass
class StepEntry:
    slot: int
    tokens: Sequence[int]
    want: Sequence[int] = ()


@dataclass
class CacheConfig:
    page_size: int = 16
    num_pages: int = 0                       # pages of every group, unless `pages_per_group` says otherwise
    max_requests: int = 4
    max_model_len: int = 0                   # 0: the model's maximum positions
    pages_per_group: Optional[Sequence[int]] = None
    fill_nan: bool = True                    # start the pools as NaN so that a stale read shows


@dataclass
class _RunPlan:
    block: Block
    context: RunContext
    need: Optional[CacheNeed]
    state_need: Optional[StateNeed]


class Model:
    def __init__(self, plan: ModelPlan, rt: Runtime):
        plan.validate()
        self.plan, self.rt = plan, rt
        self.parts = build_parts(plan)
        self.positions, self.embedding = self.parts.positions, self.parts.embedding
        self.final_norm, self.lm_head, self.blocks = self.parts.final_norm, self.parts.lm_head, self.parts.blocks
        # Cache groups: runs whose mixers keep the same span of keys share page ids.
        self.group_windows: List[Optional[int]] = []
        self.runs: List[_RunPlan] = []
        for i, run in enumerate(plan.schedule):
            block = self.blocks[run.layer]
            need, state_need = block.mixer.cache_need(), block.mixer.state_need()
            ctx = RunContext()
            if run.kv_from is not None:
                source = self.runs[run.kv_from]
                if need is None or source.need != need:
                    raise ValueError(f"run {i} cannot read the cache of run {run.kv_from}: {need} vs {source.need}")
                ctx.group, ctx.write_cache = source.context.group, False
            elif need is not None:
                if need.window not in self.group_windows:
                    self.group_windows.append(need.window)
                ctx.group = self.group_windows.index(need.window)
            self.runs.append(_RunPlan(block, ctx, need, state_need))
        self.cache: Optional[CacheManager] = None
        self.cache_config: Optional[CacheConfig] = None
        self.status = None
        self._pinned: List[Tuple[torch.Tensor, torch.cuda.Event]] = []
        self._pinned_next = 0
        self._bound = False
        self.poisoned: Optional[str] = None      # why the model refuses further work, once it does
        # For tests: called with (group, slots, table rows on the host) after a step's block table is
        # filled and before it is uploaded; it may change the rows it is given.
        self.table_hook = None
        self._hook_sent = None
        self.last_h2d_bytes = 0
        # A model whose parts all compile (`Part.compiles`) and keep no per-request state runs its steps
        # in the native executor (programs of launches, CUDA graphs for decode shapes); any other
        # model is stepped from Python, part by part, without graphs.
        self._native: Optional[NativeStepper] = None
        self._compiles = (all(r.state_need is None for r in self.runs) and all(p.compiles() for p in self._all_parts())
                          and all(b.compiles() for b in self.blocks))
        self.use_graphs = True
        # Table width of a graph, in blocks: a graph serves the contexts of one bucket, and its
        # attention launch is planned for the bucket's upper end.  Set to about 1024 tokens when
        # the cache is allocated (a wider bucket plans key splits that short contexts leave idle).
        self.graph_bucket_blocks = 64
        self.max_graphs = 48
        self.graph_after = 2        # steps of a shape that run launch by launch before the shape is captured

    # ------------------------------------------------------------------ weights
    def _all_parts(self):
        return iter(self.parts)

    def expected_weights(self) -> Dict[str, WeightSpec]:
        return merge_specs(spec for part in self._all_parts() for spec in part.weight_specs())

    def kernel_modules(self) -> List[str]:
        names = ["host", "sampling", "weights"]
        for part in self._all_parts():
            names += part.kernel_modules(self.rt.dtype)
        return list(dict.fromkeys(names))

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        build.ensure(self.kernel_modules())
        self.rt.begin_load(tensors)
        for part in self._all_parts():
            part.bind(tensors, self.rt)
        self.rt.end_load()
        self.status = torch.zeros(1, dtype=torch.int32, device=self.rt.device)
        self.rt.status = self.status
        self._bound = True

    # ------------------------------------------------------------------ cache
    def allocate_cache(self, config: CacheConfig) -> None:
        max_len = config.max_model_len or self.plan.max_positions
        if max_len > self.plan.max_positions:
            raise ValueError(f"max_model_len {max_len} exceeds the model's {self.plan.max_positions} positions")
        pages = list(config.pages_per_group) if config.pages_per_group else [config.num_pages] * len(self.group_windows)
        if len(pages) != len(self.group_windows) or any(p <= 0 for p in pages):
            raise ValueError(f"need a positive page count for each of {len(self.group_windows)} cache groups, got {pages}")
        self.cache_config = CacheConfig(config.page_size, config.num_pages, config.max_requests, max_len, pages, config.fill_nan)
        self.graph_bucket_blocks = max(1, 1024 // config.page_size)
        self.cache = CacheManager([GroupSpec(w, p) for w, p in zip(self.group_windows, pages)],
                                  config.page_size, config.max_requests, max_len)
        for i, run in enumerate(self.runs):
            ctx = run.context
            if run.need is not None and ctx.write_cache:
                shape = (pages[ctx.group], 2, run.need.kv_heads, config.page_size, run.need.head_dim)
                ctx.cache = torch.empty(shape, dtype=self.rt.dtype, device=self.rt.device)
                if config.fill_nan:
                    ctx.cache.view(torch.uint8).fill_(0xFF)   # all-ones bytes are NaN in both precisions
            if run.state_need is not None:
                ctx.state = torch.zeros((config.max_requests, *run.state_need.shape), dtype=run.state_need.dtype,
                                        device=self.rt.device)
        for i, run in enumerate(self.runs):
            source = self.plan.schedule[i].kv_from
            if source is not None:
                run.context.cache = self.runs[source].context.cache
        self._native = NativeStepper(self) if self._compiles else None

    def emit_program(self, b) -> None:
        """The whole step as the parts describe it to a program builder: embedding, the runs in the
        plan's order, the final norm over the wanted rows, the head.  The residual stream lives for
        the whole step; what a run needs is cut from two alternating banks, so the contribution a run
        leaves pending for the next norm is not overwritten by that next run."""
        h = self.embedding.emit(b)
        b.start_banks()
        pending = None
        for at, run in enumerate(self.runs):
            b.next_bank()
            following = self.runs[at + 1].block.first_norm() if at + 1 < len(self.runs) else None
            b.norm_after_block = following.foldable() if following is not None else None
            pending = run.block.emit(b, h, pending, run.context)
        b.norm_after_block = None
        b.next_bank()
        x = self.final_norm.emit(b, h, pending, True)
        self.lm_head.emit(b, x)

    @property
    def _graphs(self):
        """The decode shapes that have a CUDA graph (only their number is of interest outside)."""
        return list(range(self._native.graph_count())) if self._native is not None else []

    @property
    def graph_launches(self) -> int:
        """Launches that graph replays stood for so far."""
        return self._native.graph_launches if self._native is not None else 0

    @property
    def steady_state_allocations(self) -> int:
        """How often a buffer of the native stepper had to grow (it stops once the largest step has been seen)."""
        return self._native.allocations if self._native is not None else 0

    def cache_bytes_per_token(self) -> int:
        element = 2 if self.rt.is_bf16 else 4
        return sum(2 * r.need.kv_heads * r.need.head_dim * element for r in self.runs
                   if r.need is not None and r.context.write_cache)

    def _refuse_if_poisoned(self) -> None:
        if self.poisoned is not None:
            raise Poisoned(f"the model is poisoned and must not be used further ({self.poisoned})")

    def _poison(self, why: str) -> None:
        if self.poisoned is None:
            self.poisoned = why
            if self._native is not None:
                self._native.poison(why)

    def open_request(self) -> int:
        self._refuse_if_poisoned()
        slot = self.cache.open()
        for run in self.runs:
            if run.context.state is not None:
                run.context.state[slot].zero_()
        return slot

    def close_request(self, slot: int) -> None:
        self.cache.close(slot)

    # ------------------------------------------------------------------ the step
    def _pinned_buffer(self, count: int) -> torch.Tensor:
        if len(self._pinned) < 4:
            self._pinned.append((torch.empty(max(count, 1 << 16), dtype=torch.int32, pin_memory=True), torch.cuda.Event()))
            index = len(self._pinned) - 1
        else:
            index = self._pinned_next
            self._pinned_next = (index + 1) % len(self._pinned)
        buffer, event = self._pinned[index]
        event.synchronize()
        if buffer.numel() < count:
            buffer = torch.empty(count * 2, dtype=torch.int32, pin_memory=True)
            self._pinned[index] = (buffer, event)
        self._pinned_current = index
        return buffer

    def _validate(self, entries: Sequence[StepEntry]):
        if not self._bound or self.cache is None:
            raise StepError("the model has no weights or no cache yet")
        if not entries:
            raise StepError("a step needs at least one entry")
        segments, row = [], 0
        seen = set()
        max_len = self.cache_config.max_model_len
        for e in entries:
            count = len(e.tokens)
            if count == 0:
                raise StepError(f"the entry of slot {e.slot} has no tokens")
            if e.slot in seen:
                raise StepError(f"slot {e.slot} appears twice in one step")
            seen.add(e.slot)
            start = self.cache.length(e.slot)
            if start + count > max_len:
                raise StepError(f"slot {e.slot} would hold {start + count} tokens, the limit is {max_len}")
            for w in e.want:
                if not 0 <= w < count:
                    raise StepError(f"slot {e.slot} wants logits at place {w} of {count} tokens")
            segments.append(Segment(e.slot, start, count, row))
            row += count
        return segments, row

    def step(self, entries: Sequence[StepEntry], device_tokens: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
        """Runs the entries' tokens as one batch from the cache and returns the float32
        logits [wanted, vocab] in the order of the entries and of each entry's `want`
        (None if nothing is wanted).  Raises `OutOfPages` before any device work if
        the cache cannot hold the step.

        `device_tokens` (int32 on the device, one id per row) replaces the entries'
        token values, whose count still says how many rows each entry brings: a
        decode loop can feed sampled ids back without a round trip to the host.

        A step of single tokens that wants every row's logits is replayed from a CUDA
        graph (captured when its batch size and context bucket come for the third time).
        The logits live in a buffer that the next step writes again: read or sample them
        before the next step.

        Failure: a batch that is refused, or a pool that cannot hold it, raises before any
        device work and changes nothing.  An exception after device work has begun rolls the
        ledger back (the step's pages, lengths, and the fixed-size state of its requests as
        they were before the step), poisons the model and is raised again."""
        self._refuse_if_poisoned()
        if not self._bound or self.cache is None:
            raise StepError("the model has no weights or no cache yet")
        if self._native is not None:
            return self._native_step(entries, device_tokens)
        return self._python_step(entries, device_tokens)

    def _native_step(self, entries: Sequence[StepEntry], device_tokens: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
        """The step in the native executor: everything from the validation of the entries to the
        publishing of lengths happens in `mlr_model_step`; this only hands over the entries."""
        native_model = self._native
        if not entries:
            raise StepError("a step needs at least one entry")
        slots = [e.slot for e in entries]
        counts = [len(e.tokens) for e in entries]
        offsets, places = [0], []
        for e in entries:
            places.extend(e.want)
            offsets.append(len(places))
        rows = sum(counts)
        tokens = None
        if device_tokens is None:
            tokens = np.concatenate([np.asarray(e.tokens, dtype=np.int64) for e in entries]) if rows else np.zeros(0, np.int64)
            if rows and (tokens.min() < 0 or tokens.max() >= self.plan.vocab_size):
                raise StepError(f"a token id is outside the vocabulary of {self.plan.vocab_size}")
            tokens = np.ascontiguousarray(tokens, dtype=np.int32)
        elif device_tokens.dtype is not torch.int32 or device_tokens.numel() != rows or not device_tokens.is_cuda:
            raise StepError("device_tokens must be int32 on the device with one id per row of the step")
        native_model.set_graphs(self.use_graphs, self.graph_after, self.graph_bucket_blocks, self.max_graphs)
        if (self.table_hook is None) != (native_model._hook is None) or self.table_hook is not self._hook_sent:
            native_model.set_table_hook(self.table_hook)
            self._hook_sent = self.table_hook
        from ..ops import native
        code, message, logits = native_model.step(slots, counts, tokens, offsets, places, device_tokens, native.stream())
        self.last_h2d_bytes = int(native_model.last_info.h2d_bytes)
        if code == STEP_OK:
            return logits
        if code == STEP_REFUSED:
            raise StepError(message)
        if code == STEP_NO_PAGES:
            raise OutOfPages(message)
        if code == STEP_POISONED:
            raise Poisoned(message)
        self.poisoned = self.poisoned or message
        raise native.KernelError(message)

    def _python_step(self, entries: Sequence[StepEntry], device_tokens: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
        """The step driven from Python, for models with parts that do not compile into programs:
        the same order of work (validate, take pages, pack and upload the metadata, run the parts,
        publish), every part through its `forward`.  No CUDA graphs on this path."""
        segments, rows = self._validate(entries)
        n = len(segments)
        vocab = self.plan.vocab_size
        tokens = np.concatenate([np.asarray(e.tokens, dtype=np.int64) for e in entries])
        if device_tokens is None and (tokens.min() < 0 or tokens.max() >= vocab):
            raise StepError(f"a token id is outside the vocabulary of {vocab}")
        if device_tokens is not None and (device_tokens.dtype is not torch.int32 or device_tokens.numel() != rows):
            raise StepError("device_tokens must be int32 with one id per row of the step")
        want_rows = [s.row + w for s, e in zip(segments, entries) for w in e.want]
        all_single = all(s.count == 1 for s in segments)
        self.cache.prepare([s.slot for s in segments], [s.count for s in segments])
        try:
            page = self.cache_config.page_size
            max_context = max(s.start + s.count for s in segments)
            columns = (max_context + page - 1) // page
            n_groups = len(self.group_windows)
            # One packed int32 buffer: ids | positions | segment_of_row | info[n,4] | slots | want | tables
            sizes = [rows, rows, rows, 4 * n, n, len(want_rows)] + [n * columns] * n_groups
            offsets = np.concatenate([[0], np.cumsum(sizes)])
            total = int(offsets[-1])
            host = self._pinned_buffer(total)
            view = host.numpy()
            view[offsets[0]:offsets[1]] = tokens
            for i, s in enumerate(segments):
                view[offsets[1] + s.row: offsets[1] + s.row + s.count] = np.arange(s.start, s.start + s.count)
                view[offsets[2] + s.row: offsets[2] + s.row + s.count] = i
                view[offsets[3] + 4 * i: offsets[3] + 4 * i + 4] = (s.row, s.count, s.start, s.slot)
                view[offsets[4] + i] = s.slot
            view[offsets[5]:offsets[6]] = want_rows
            slots = [s.slot for s in segments]
            for g in range(n_groups):
                table = host[offsets[6 + g]:offsets[7 + g]].view(n, columns)
                self.cache.fill_table(g, slots, table, min(columns, self.cache.max_blocks))
                if self.table_hook is not None:
                    self.table_hook(g, slots, table)
            self.last_h2d_bytes = 4 * total
        except BaseException:
            self.cache.discard()        # nothing has been launched: the model stays usable
            raise
        journal = None
        try:
            journal = self._journal_state(slots)
            device = torch.empty(total, dtype=torch.int32, device=self.rt.device)
            device.copy_(host[:total], non_blocking=True)
            self._pinned[self._pinned_current][1].record()
            if device_tokens is not None:
                device[:rows].copy_(device_tokens)
            part = lambda k: device[offsets[k]:offsets[k + 1]]
            step = StepContext(
                rt=self.rt, num_rows=rows, segments=segments, token_ids=part(0), positions=part(1),
                segment_of_row=part(2), segment_info=part(3).view(n, 4), slots=part(4),
                tables={g: part(6 + g).view(n, columns) for g in range(n_groups)},
                page_size=page, status=self.status, max_count=max(s.count for s in segments),
                max_context=max_context, all_single=all_single, context_bound=None)
            logits = self._forward(step, part(5) if want_rows else None)
        except BaseException as error:
            self._poison(f"a step failed after its device work had begun: {type(error).__name__}: {error}")
            try:
                self._restore_state(journal)
            finally:
                self.cache.discard()
            raise
        # Lengths and page maps are published when the step's work is enqueued, not when it has run,
        # so that the next step can be launched behind it.  A fault a kernel reports in the status
        # word is read with the step's results (`check_status`, or the engine's read-back) and poisons
        # the model before any token of that step is handed out.
        self.cache.commit()
        return logits

    def _journal_state(self, slots: Sequence[int]):
        """Copies of the fixed-size state of the step's requests, for runs that keep one: a mixer
        updates its state in place, and a step that fails must not leave it half updated."""
        saved = [(run.context.state, slot, run.context.state[slot].clone())
                 for run in self.runs if run.context.state is not None for slot in slots]
        return saved or None

    def _restore_state(self, journal) -> None:
        for state, slot, saved in journal or ():
            state[slot].copy_(saved)

    def _forward(self, step: StepContext, want_rows: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
        h = self.embedding.forward(step)
        for position in self.positions.values():
            position.add_to_embedding(h, step)
        pending = None
        for run in self.runs:
            pending = run.block.forward(h, pending, step, run.context)
        if want_rows is None:
            return None
        x = self.final_norm.forward(h, pending, step, rows=want_rows)
        return self.lm_head.forward(x, step)

    def check_status(self) -> None:
        """Reads the device status word (this waits for the device) and raises if a
        kernel flagged a fault.  After a fault the model must not be used further."""
        value = int(self.status.item())
        if value:
            self._poison(f"kernels reported status {value}")
            raise DeviceFault(f"kernels reported status {value} (1 = index outside a table, 2 = page outside the pool, "
                              f"4 = non-finite logits); the cache can no longer be trusted")
