"""Shared by the GPU tests: tiny model folders, the engine on them, comparisons."""
from __future__ import annotations

import json
import os
from typing import Dict, List, Optional, Sequence

import torch

import plain_qwen3
import tiny_models


def write_model_folder(folder: str, config: dict, weights: Dict[str, torch.Tensor]) -> None:
    from mini_llm_runtime_b200.weights.safetensors_io import write_safetensors
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(config, f)
    write_safetensors(os.path.join(folder, "model.safetensors"), weights)


def tiny_folder(tmp_path_factory, name: str, seed: int):
    """A folder with config `name` and bf16-rounded random weights; returns
    (folder, config dict, weights dict)."""
    config = tiny_models.get(name)
    weights = plain_qwen3.random_weights(config, seed)
    folder = str(tmp_path_factory.mktemp(name))
    write_model_folder(folder, config, weights)
    return folder, config, weights


def random_tokens(config: dict, count: int, seed: int) -> List[int]:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, config["vocab_size"], (count,), generator=g).tolist()


def engine_model(folder: str, dtype: str, num_pages: int, page_size: int = 16, max_requests: int = 4):
    from mini_llm_runtime_b200.engine.loading import load_model
    from mini_llm_runtime_b200.engine.model import CacheConfig
    return load_model(folder, dtype, CacheConfig(page_size=page_size, num_pages=num_pages, max_requests=max_requests))


def run_whole(model, tokens: Sequence[int]) -> torch.Tensor:
    """One request, all tokens in one step, logits at every position."""
    from mini_llm_runtime_b200.engine.model import StepEntry
    slot = model.open_request()
    logits = model.step([StepEntry(slot, list(tokens), list(range(len(tokens))))])
    model.check_status()
    model.close_request(slot)
    return logits.float().cpu()


def run_portions(model, tokens: Sequence[int], sizes: Sequence[int]) -> torch.Tensor:
    """One request cut into portions of the given sizes (the last size repeats)."""
    from mini_llm_runtime_b200.engine.model import StepEntry
    slot = model.open_request()
    out, pos, i = [], 0, 0
    while pos < len(tokens):
        n = min(sizes[min(i, len(sizes) - 1)], len(tokens) - pos)
        out.append(model.step([StepEntry(slot, list(tokens[pos:pos + n]), list(range(n)))]).float().cpu())
        pos += n
        i += 1
    model.check_status()
    model.close_request(slot)
    return torch.cat(out)


# Tolerances: float32 results differ from the plain implementation by summation order
# only; bfloat16 results carry the rounding of activations and cache to 8 bits of
# mantissa at every layer.
TOL = {"float32": dict(atol=2e-4, rtol=2e-4), "bfloat16": dict(atol=6e-2, rtol=6e-2)}


def assert_close(got: torch.Tensor, want: torch.Tensor, dtype: str, what: str = "") -> None:
    tol = TOL[dtype]
    assert got.shape == want.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(want.shape)}"
    assert torch.isfinite(got).all(), f"{what}: non-finite values"
    diff = (got - want).abs()
    bound = tol["atol"] + tol["rtol"] * want.abs()
    if not (diff <= bound).all():
        bad = torch.nonzero(diff > bound)
        first = bad[0].tolist()
        raise AssertionError(f"{what}: {len(bad)} of {diff.numel()} values differ; first at {first} "
                             f"(row = position): got {got[tuple(first)]:.6f}, want {want[tuple(first)]:.6f}; "
                             f"max abs diff {diff.max():.3e}")
