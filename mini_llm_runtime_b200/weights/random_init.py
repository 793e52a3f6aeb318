"""Random-weights mode: tensors for a model from its weight specs and a seed.

`write_random_model` writes a model folder (config.json, model.safetensors) that the
normal loading path reads back; `random_tensors` makes the same tensors in memory.
Matrices are N(0, 0.02^2), norm weights 1 + N(0, 0.01^2), rounded once to float32 and
once to the stored dtype.  The reference has a fixture of this kind only in its tests
(tests/qwen3_fixture.h:10-82).

A tensor's numbers depend on (seed, tensor name, element index) and on nothing else: the
generator (`portable_random.py`) is counter based and made of exactly defined operations,
so numpy on a host and the kernel `mlr_normal_fill` on the GPU give the same bits.  A
model made on the device for a measurement and the folder `--random-weights` writes for
the same seed therefore hold the same tensors.
"""
from __future__ import annotations

import json
import os
from typing import Dict

import numpy as np
import torch

from .loader import WeightSpec
from .portable_random import normal_float32, tensor_key
from .safetensors_io import write_safetensors

_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32}


def _rule(name: str, spec: WeightSpec):
    kind, std = spec.init
    if kind not in ("normal", "one_plus_normal"):
        raise ValueError(f"tensor {name!r} has unknown init rule {kind!r}")
    return kind == "one_plus_normal", float(std)


def random_tensor(name: str, spec: WeightSpec, seed: int, dtype: torch.dtype, device: str = "cpu") -> torch.Tensor:
    one_plus, std = _rule(name, spec)
    count = int(np.prod(spec.shape)) if len(spec.shape) else 1
    if torch.device(device).type == "cpu":
        values = normal_float32(seed, name, count, std, one_plus)
        return torch.from_numpy(values).view(*spec.shape).to(dtype)
    from ..ops import native
    out = torch.empty(spec.shape, dtype=dtype, device=device)
    with torch.cuda.device(out.device):
        native.call("weights", "mlr_normal_fill", out.data_ptr(), native.is_bf16(out), count,
                    tensor_key(seed, name), std, int(one_plus), native.stream())
    return out


def random_tensors(specs: Dict[str, WeightSpec], seed: int, dtype: torch.dtype = torch.bfloat16,
                   device: str = "cpu") -> Dict[str, torch.Tensor]:
    if dtype not in (torch.bfloat16, torch.float32):
        raise ValueError("random weights are stored as bfloat16 or float32")
    return {name: random_tensor(name, specs[name], seed, dtype, device) for name in sorted(specs)}


def write_random_model(model_dir: str, config: dict, seed: int, dtype: str = "bfloat16", device: str = "cpu") -> None:
    """Writes `config.json` and `model.safetensors` for `config` (a config.json
    dictionary of a registered architecture).  `device`: where the numbers are made
    (the file is the same either way; a GPU makes a large model in seconds)."""
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
    tensors = {n: t.cpu() for n, t in random_tensors(specs, seed, _DTYPES[dtype], device).items()}
    write_safetensors(os.path.join(model_dir, "model.safetensors"), tensors, {"format": "pt", "seed": str(seed)})
