"""Random-weights mode: tensors for a model from its weight specs and a seed.

`write_random_model` writes a model folder (config.json, model.safetensors) that the
normal loading path reads back; `random_tensors` makes the same tensors in memory
(on a GPU for sizes that would take minutes on the host).  Matrices are
N(0, 0.02^2), norm weights 1 + N(0, 0.01^2), rounded once to the stored dtype.  The
reference has a fixture of this kind only in its tests (tests/qwen3_fixture.h:10-82).

Tensors are drawn in sorted name order from one generator, so a seed, a device and
a set of specs give the same tensors every time.  Host and GPU generators differ:
the folder written on one machine is the portable artefact, not the seed.
"""
from __future__ import annotations

import json
import os
from typing import Dict

import torch

from .loader import WeightSpec
from .safetensors_io import write_safetensors

_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32}


def random_tensors(specs: Dict[str, WeightSpec], seed: int, dtype: torch.dtype = torch.bfloat16,
                   device: str = "cpu") -> Dict[str, torch.Tensor]:
    generator = torch.Generator(device=device).manual_seed(seed)
    out = {}
    for name in sorted(specs):
        spec = specs[name]
        kind, std = spec.init
        t = torch.randn(spec.shape, generator=generator, dtype=torch.float32, device=device) * std
        if kind == "one_plus_normal":
            t += 1.0
        elif kind != "normal":
            raise ValueError(f"tensor {name!r} has unknown init rule {kind!r}")
        out[name] = t.to(dtype)
    return out


def write_random_model(model_dir: str, config: dict, seed: int, dtype: str = "bfloat16") -> None:
    """Writes `config.json` and `model.safetensors` for `config` (a config.json
    dictionary of a registered architecture)."""
    from ..config.registry import config_from_dict, plan_for
    from ..engine.structure import expected_weights

    if dtype not in _DTYPES:
        raise ValueError(f"dtype must be one of {sorted(_DTYPES)}")
    specs = expected_weights(plan_for(config_from_dict(config)))
    os.makedirs(model_dir, exist_ok=True)
    stored = dict(config)
    stored["torch_dtype"] = dtype
    with open(os.path.join(model_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(stored, f, indent=2)
    write_safetensors(os.path.join(model_dir, "model.safetensors"),
                      random_tensors(specs, seed, _DTYPES[dtype]), {"format": "pt", "seed": str(seed)})
