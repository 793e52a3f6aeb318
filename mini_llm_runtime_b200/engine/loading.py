"""From a model folder to a model that can step."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import models as _models  # noqa: F401  (registers the architectures)
from ..config.registry import config_from_dict, config_from_dir, plan_for
from ..weights.loader import load_checkpoint
from ..weights.random_init import random_tensors
from .model import CacheConfig, Model
from .runtime import Runtime

DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32}


def parse_dtype(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        return name
    try:
        return DTYPES[name]
    except KeyError:
        raise ValueError(f"dtype must be one of {sorted(DTYPES)}, got {name!r}") from None


def load_model(model_dir: str, dtype="bfloat16", cache: Optional[CacheConfig] = None, device: str = "cuda:0") -> Model:
    """Reads config.json, picks the architecture from the registry, checks and loads
    the weights by name, and allocates the cache."""
    config = config_from_dir(model_dir)
    plan = plan_for(config)
    model = Model(plan, Runtime(parse_dtype(dtype), device))
    model.config = config
    tensors = load_checkpoint(model_dir, model.expected_weights(), plan.redundant_tensors)
    model.bind(tensors)
    if cache is not None:
        model.allocate_cache(cache)
    return model


def random_model(config: dict, seed: int, dtype="bfloat16", cache: Optional[CacheConfig] = None,
                 device: str = "cuda:0") -> Model:
    """A model of `config` with seeded random weights made on the device, without a
    folder in between (for measurements at sizes where writing one is pointless)."""
    cfg = config_from_dict(config)
    plan = plan_for(cfg)
    model = Model(plan, Runtime(parse_dtype(dtype), device))
    model.config = cfg
    tensors = random_tensors(model.expected_weights(), seed, torch.bfloat16, device)
    model.bind(tensors)
    del tensors
    if cache is not None:
        model.allocate_cache(cache)
    return model
