"""Data that describes a model: part specifications, layers, the run order.

An architecture is described to the engine as a `ModelPlan`.  The plan holds no
code: each part is a `PartSpec` (a registered kind plus its sizes and constants),
each layer a `LayerSpec` (which block arrangement, which mixer, which feed-forward,
which norms), and the order in which layers run is a list of `Run` entries.  The
generic model in `engine/model.py` builds itself from a plan; an architecture
module only translates its own config.json into one.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple


class ConfigError(ValueError):
    """A config.json that this engine cannot run, with the reason."""


@dataclass(frozen=True)
class PartSpec:
    """A registered part kind with its parameters.

    `params` holds every size and constant of the part (nothing is read from a
    global config later).  `weights` maps the part's own role names ("q", "gate",
    "weight", ...) to full checkpoint tensor names.
    """
    kind: str
    params: Dict[str, Any] = field(default_factory=dict)
    weights: Dict[str, str] = field(default_factory=dict)


@dataclass(frozen=True)
class LayerSpec:
    """One layer: a block arrangement around a mixer and a feed-forward.

    `norms` maps the arrangement's norm slots (for the pre-norm block:
    "pre_mixer", "pre_feed_forward") to norm specs.
    """
    block: str
    mixer: PartSpec
    feed_forward: PartSpec
    norms: Dict[str, PartSpec]


@dataclass(frozen=True)
class Run:
    """One entry of the run order.

    `layer` indexes `ModelPlan.layers`; a layer may be named by several runs and
    then runs again with the same weights and a cache of its own.  `kv_from`, when
    set, is the index of an earlier run whose cache this run reads instead of
    writing one.
    """
    layer: int
    kv_from: Optional[int] = None


@dataclass(frozen=True)
class ModelPlan:
    architecture: str
    hidden_size: int
    vocab_size: int
    max_positions: int
    embedding: PartSpec
    positions: Dict[str, PartSpec]
    layers: Tuple[LayerSpec, ...]
    schedule: Tuple[Run, ...]
    final_norm: PartSpec
    lm_head: PartSpec
    eos_token_ids: Tuple[int, ...] = ()
    # (name, twin): a checkpoint may also store `name`, a second copy of the tensor `twin` that the
    # model reads (a tied output head stored beside the embedding).  It is accepted if it equals its twin.
    redundant_tensors: Tuple[Tuple[str, str], ...] = ()

    def validate(self) -> None:
        if not self.layers or not self.schedule:
            raise ConfigError("a model plan needs at least one layer and one run")
        for i, run in enumerate(self.schedule):
            if not 0 <= run.layer < len(self.layers):
                raise ConfigError(f"run {i} names layer {run.layer}, the plan has {len(self.layers)}")
            if run.kv_from is not None:
                if not 0 <= run.kv_from < i:
                    raise ConfigError(f"run {i} reads the cache of run {run.kv_from}, which is not an earlier run")
                if self.schedule[run.kv_from].kv_from is not None:
                    raise ConfigError(f"run {i} reads the cache of run {run.kv_from}, which owns none")
        for layer in self.layers:
            pos = layer.mixer.params.get("position")
            if pos is not None and pos not in self.positions:
                raise ConfigError(f"mixer names position encoding {pos!r}, the plan has {sorted(self.positions)}")
