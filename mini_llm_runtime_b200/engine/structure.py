"""The parts of a plan, built in one place.

Parts are built from their specs alone, so the expected tensor names and shapes of a plan can
be listed on any machine (the loader's errors and the random-weights writer use this), and the
generic model (`engine/model.py`) gets its parts from the same function: there is one traversal
of a plan, and a new category of part is added here and in the registry.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Iterator, List

from .. import parts as _builtin_parts  # noqa: F401
from ..config.base import ModelPlan, PartSpec
from ..config.registry import part_class
from ..parts.base import Block, Part
from ..weights.loader import WeightSpec, merge_specs


def build_part(category: str, spec: PartSpec):
    return part_class(category, spec.kind)(spec)


@dataclass
class BuiltParts:
    embedding: Part
    positions: Dict[str, Part]
    blocks: List[Block]
    final_norm: Part
    lm_head: Part

    def __iter__(self) -> Iterator[Part]:
        """Every part once, in the order of the computation."""
        yield self.embedding
        yield from self.positions.values()
        for block in self.blocks:
            yield block.mixer
            yield block.feed_forward
            yield from block.norms.values()
        yield self.final_norm
        yield self.lm_head


def build_parts(plan: ModelPlan) -> BuiltParts:
    positions = {name: build_part("position", spec) for name, spec in plan.positions.items()}
    blocks = []
    for layer in plan.layers:
        mixer = build_part("mixer", layer.mixer)
        if getattr(mixer, "position_name", None) is not None:
            mixer.position = positions[mixer.position_name]
        feed_forward = build_part("feed_forward", layer.feed_forward)
        norms = {slot: build_part("norm", spec) for slot, spec in layer.norms.items()}
        blocks.append(part_class("block", layer.block)(PartSpec(layer.block), mixer, feed_forward, norms))
    return BuiltParts(build_part("embedding", plan.embedding), positions, blocks, build_part("norm", plan.final_norm),
                      build_part("lm_head", plan.lm_head))


def expected_weights(plan: ModelPlan) -> Dict[str, WeightSpec]:
    return merge_specs(spec for part in build_parts(plan) for spec in part.weight_specs())
