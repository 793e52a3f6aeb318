"""What a plan needs from a checkpoint, worked out without a GPU.

Parts declare their tensors from their specs alone, so the expected names and
shapes can be listed on any machine; the loader's errors and the random-weights
writer use this.
"""
from __future__ import annotations

from typing import Dict

from .. import parts as _builtin_parts  # noqa: F401
from ..config.base import ModelPlan
from ..config.registry import part_class
from ..weights.loader import WeightSpec, merge_specs


def expected_weights(plan: ModelPlan) -> Dict[str, WeightSpec]:
    specs = []
    specs += part_class("embedding", plan.embedding.kind)(plan.embedding).weight_specs()
    for spec in plan.positions.values():
        specs += part_class("position", spec.kind)(spec).weight_specs()
    for layer in plan.layers:
        specs += part_class("mixer", layer.mixer.kind)(layer.mixer).weight_specs()
        specs += part_class("feed_forward", layer.feed_forward.kind)(layer.feed_forward).weight_specs()
        for norm in layer.norms.values():
            specs += part_class("norm", norm.kind)(norm).weight_specs()
    specs += part_class("norm", plan.final_norm.kind)(plan.final_norm).weight_specs()
    specs += part_class("lm_head", plan.lm_head.kind)(plan.lm_head).weight_specs()
    return merge_specs(specs)
