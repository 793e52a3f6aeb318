"""Interfaces of the parts a layer is put together from, and what a step hands them.

A part is built from a `PartSpec` alone (its sizes and constants are the spec's
parameters), declares the checkpoint tensors it needs, is bound to them once, and
is then called once per step for all rows of the batch.  No part knows which model
it is in, which layer it is, or what the other layers are.

    Mixer          forward(x, step, run) -> delta      tokens exchange information
    FeedForward    forward(x, step) -> delta           per-token
    Norm           forward(h, delta, ...) -> x         also moves the residual stream on
    PositionEncoding   rotation_table() / add_to_embedding(h, step)
    Block          forward(h, pending, step, run) -> pending     arranges the above

`x` is [M, width] in the activation dtype; `h` is the float32 residual stream;
`delta` is a float32 [M, width] contribution that has not been added to `h` yet.

A part says what it does in one of two ways.  A part written with torch operations overrides
`forward` (tensors in, tensors out); the model then runs its steps from Python.  A part made
of this package's kernels overrides `emit(builder, ...)` instead (buffers of the builder in
and out, see `engine/builder.py`): it lists its launches, and `forward` is the default that
runs that list at once.  When every part of a model has an `emit`, the model compiles them
into programs that the native executor walks without Python (`Part.compiles`).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ..config.base import PartSpec
from ..weights.loader import WeightSpec


# --------------------------------------------------------------------------- needs
@dataclass(frozen=True)
class CacheNeed:
    """A mixer that keeps keys and values per token: how far back it reads
    (`window` None = everything) and the page geometry of one layer."""
    window: Optional[int]
    kv_heads: int
    head_dim: int


@dataclass(frozen=True)
class StateNeed:
    """A mixer that keeps a state of fixed size per request (`shape` without the
    request dimension).  A new request starts from zeros."""
    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


# --------------------------------------------------------------------------- what a step carries
@dataclass(frozen=True)
class Segment:
    """The rows one request contributes to a step: `count` consecutive tokens from
    position `start`, at rows [row, row + count) of the batch."""
    slot: int
    start: int
    count: int
    row: int


@dataclass
class StepContext:
    """Everything about a step that parts may read.  Device tensors are int32."""
    rt: "object"                      # engine.runtime.Runtime
    num_rows: int
    segments: List[Segment]           # host copy, in batch order
    token_ids: torch.Tensor           # [M]
    positions: torch.Tensor           # [M]
    segment_of_row: torch.Tensor      # [M] index into `segments`
    segment_info: torch.Tensor        # [n_segments, 4]: first row, count, start position, slot
    slots: torch.Tensor               # [n_segments] state slot of each segment
    tables: Dict[int, torch.Tensor]   # cache group -> block table rows [n_segments, columns]
    page_size: int
    status: torch.Tensor              # [1] device status word
    max_count: int = 0                # longest segment of the step
    max_context: int = 0              # largest position + 1 of the step
    all_single: bool = False          # every segment is one token (a pure decode step)
    context_bound: Optional[int] = None   # set when the step is captured into a CUDA graph: launch shapes
                                          # must be planned for contexts up to this bound, not for the
                                          # lengths of the step at hand
    scratch: Dict[str, object] = field(default_factory=dict)   # per-step memo for kernels' plans
    # The float32 residual stream while a block runs.  A mixer or feed-forward whose last
    # product can add its result straight into it (h += x W^T in the product's epilogue)
    # does so and returns None instead of a contribution for the next norm to add.
    residual: Optional[torch.Tensor] = None


@dataclass
class RunContext:
    """What one entry of the run order gives its mixer."""
    group: Optional[int] = None           # cache group of this run's mixer
    cache: Optional[torch.Tensor] = None  # [pages, 2, kv_heads, page_size, head_dim]
    write_cache: bool = True              # False: the run reads a cache another run writes
    state: Optional[torch.Tensor] = None  # [max_requests, *StateNeed.shape]


# --------------------------------------------------------------------------- parts
class Part:
    category = ""
    # Whether `forward` may be captured in a CUDA graph and replayed: it launches the same
    # kernels with the same shapes for every step of a given batch size, reads nothing back
    # to the host and keeps no state that a repeated run would advance twice.  A model with
    # a part that says False launches its decode steps kernel by kernel.
    graph_safe = True

    def __init__(self, spec: PartSpec):
        self.spec = spec

    def weight_specs(self) -> List[WeightSpec]:
        return []

    def kernel_modules(self, dtype: torch.dtype) -> List[str]:
        """Kernel modules this part launches in the given precision (built before the
        first step)."""
        return []

    def bind(self, tensors: Dict[str, torch.Tensor], rt) -> None:
        """Takes its tensors (CPU or device, stored precision) and keeps device copies
        in the form its kernels want."""

    def emit(self, b, *args):
        """The part's launches, listed to a builder.  Parts written in torch do not have one."""
        raise NotImplementedError

    def compiles(self) -> bool:
        """Whether the native executor may run this part from `emit`: its class brings an `emit`
        and leaves `forward` as the default that runs `emit` at once."""
        return _definer(type(self), "emit") not in _INTERFACES and _definer(type(self), "forward") in _INTERFACES


def _definer(cls, name):
    for k in cls.__mro__:
        if name in k.__dict__:
            return k
    return None


def _tensor_of(buf, b=None):
    if buf is None:
        return None
    if buf.norm is not None:            # a norm that waited for a product to take it: a caller in Python wants the tensor
        buf = b.rt.materialize(b, buf)
    return buf.tensor


class Mixer(Part):
    category = "mixer"

    def cache_need(self) -> Optional[CacheNeed]:
        return None

    def state_need(self) -> Optional[StateNeed]:
        return None

    def forward(self, x: torch.Tensor, step: StepContext, run: RunContext) -> torch.Tensor:
        from ..engine.builder import EagerBuilder
        b = EagerBuilder(step, residual=step.residual)
        return _tensor_of(self.emit(b, b.wrap(x), run))


class FeedForward(Part):
    category = "feed_forward"

    def forward(self, x: torch.Tensor, step: StepContext) -> torch.Tensor:
        from ..engine.builder import EagerBuilder
        b = EagerBuilder(step, residual=step.residual)
        return _tensor_of(self.emit(b, b.wrap(x)))


class Norm(Part):
    category = "norm"

    def forward(self, h: torch.Tensor, delta: Optional[torch.Tensor], step: StepContext,
                rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Adds `delta` into `h` (if given), then returns norm(h) in the activation
        dtype.  With `rows` only those rows are normed and returned (h is then left
        as it is).  `emit(b, h, delta, wanted_only)` is the same on buffers; the wanted
        rows are then the step's (`b.meta("want_rows")`, `b.want` of them)."""
        from ..engine.builder import EagerBuilder
        b = EagerBuilder(step, want_rows=rows)
        return _tensor_of(self.emit(b, b.wrap(h), b.wrap(delta), rows is not None), b)

    def foldable(self):
        """What a product needs to know to do this norm's work itself ("rms", weight, eps, width), or
        None: then the norm is always a launch of its own."""
        return None


class PositionEncoding(Part):
    category = "position"

    def rotation_table(self) -> Optional[torch.Tensor]:
        """[max_positions, rotary_dim] float32, cos in the first half of a row and sin
        in the second, for mixers that rotate q and k; None if this encoding does not
        rotate."""
        return None

    def add_to_embedding(self, h: torch.Tensor, step: StepContext) -> None:
        """Hook for encodings that act on the embedded tokens; default: nothing."""

    def compiles(self) -> bool:
        """An encoding that only supplies a rotation table launches nothing of its own."""
        return _definer(type(self), "add_to_embedding") is PositionEncoding


class Block(Part):
    category = "block"

    def __init__(self, spec: PartSpec, mixer: Mixer, feed_forward: FeedForward, norms: Dict[str, Norm]):
        super().__init__(spec)
        self.mixer, self.feed_forward, self.norms = mixer, feed_forward, norms

    def forward(self, h: torch.Tensor, pending: Optional[torch.Tensor], step: StepContext,
                run: RunContext) -> Optional[torch.Tensor]:
        """Runs the layer on the residual stream `h` with a not yet added contribution
        `pending`; returns the contribution it leaves pending.  `emit(b, h, pending, run)`
        arranges the parts' `emit`s the same way."""
        raise NotImplementedError

    def first_norm(self) -> Optional[Norm]:
        """The norm this block applies to the residual stream first, if it starts with one: the block before
        it may then prepare it (`norm_after_block` of the builder)."""
        return None

    def compiles(self) -> bool:
        return (_definer(type(self), "emit") not in _INTERFACES and self.mixer.compiles() and self.feed_forward.compiles()
                and all(n.compiles() for n in self.norms.values()))


class Embedding(Part):
    category = "embedding"

    def forward(self, step: StepContext) -> torch.Tensor:
        """The float32 residual stream [M, width] of the step's tokens; `emit(b)` on buffers."""
        from ..engine.builder import EagerBuilder
        return _tensor_of(self.emit(EagerBuilder(step)))


class Head(Part):
    category = "lm_head"

    def forward(self, x: torch.Tensor, step: StepContext) -> torch.Tensor:
        """float32 logits [rows of x, vocab]; `emit(b, x)` on buffers (the logits buffer is `b.logits`)."""
        from ..engine.builder import EagerBuilder
        b = EagerBuilder(step)
        b.want = x.shape[0]
        return _tensor_of(self.emit(b, b.wrap(x)))


_INTERFACES = (Part, Mixer, FeedForward, Norm, PositionEncoding, Block, Embedding, Head)
