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


# Tolerances.  float32 results differ from the plain implementation by summation order only:
# an absolute-plus-relative bound per value.  bfloat16 results carry the rounding of
# activations and cache to 8 bits of mantissa at every layer; they are judged row by row
# (a row = the logits of one position), relative to the size of the row's logits, in the
# manner of the reference's validation thresholds (tests/data/qwen3_validation_cases.json:41-47:
# RMSE, largest difference and cosine together):
#   rmse    root mean square of the differences / root mean square of the wanted logits
#   max     largest difference / root mean square of the wanted logits
#   cosine  of the two rows
# The bounds stand a factor of two above what the kernels deliver: on the tiny models of these
# tests the worst rows measure 0.0077 / 0.027 / 0.99997, at the layer sizes of real models
# (tests/test_real_sizes.py, wider sums and larger logits) 0.012 / 0.060 / 0.99993.  The figures of a
# run are written to the file MLR_TEST_METRICS names.  Two pages of a request in the wrong order
# move a row by more than the bounds allow (tests/test_mutation.py).
TOL = {"float32": dict(atol=2e-4, rtol=2e-4)}
BF16_BOUNDS = dict(rmse=0.015, max=0.055, cosine=0.99994)
BF16_BOUNDS_REAL_SIZES = dict(rmse=0.025, max=0.12, cosine=0.99985)


def tie_margin(row: torch.Tensor, dtype: str) -> float:
    """How far apart two logits of `row` (the plain implementation's) must be before the engine
    has to order them the same way: nothing in float32 beyond its tolerance, twice the bound on
    a single logit's error in bfloat16."""
    if dtype == "float32":
        return 2 * (TOL["float32"]["atol"] + TOL["float32"]["rtol"] * float(row.abs().max()))
    return 2 * BF16_BOUNDS["max"] * float(row.double().pow(2).mean().sqrt())


def assert_greedy_tokens(config: dict, weights: dict, prompt: Sequence[int], got: Sequence[int], dtype: str,
                         what: str = "") -> None:
    """Every generated token against the plain implementation run on the engine's own tokens
    so far: it must be the plain argmax, or lie within `tie_margin` of it."""
    tokens = list(prompt)
    for step, token in enumerate(got):
        row = plain_qwen3.forward(config, weights, tokens)[-1]
        best = plain_qwen3.greedy(row)
        if token != best:
            gap = float(row[best] - row[token])
            assert gap <= tie_margin(row, dtype), (f"{what}: token {step} is {token}, the plain implementation says {best} "
                                                   f"({gap:.4f} above it; a tie is within {tie_margin(row, dtype):.4f})")
        tokens.append(token)


def row_metrics(got: torch.Tensor, want: torch.Tensor) -> Dict[str, torch.Tensor]:
    """Per row of [rows, vocab]: relative RMSE, relative largest difference, cosine."""
    got, want = got.double(), want.double()
    diff = got - want
    size = want.pow(2).mean(-1).sqrt().clamp_min(1e-30)
    cosine = (got * want).sum(-1) / (got.norm(dim=-1) * want.norm(dim=-1)).clamp_min(1e-30)
    return {"rmse": diff.pow(2).mean(-1).sqrt() / size, "max": diff.abs().amax(-1) / size, "cosine": cosine}


def _note(what: str, dtype: str, metrics: Dict[str, torch.Tensor]) -> None:
    path = os.environ.get("MLR_TEST_METRICS")
    if path:
        with open(path, "a") as f:
            f.write(f"{dtype}\t{what}\trmse {metrics['rmse'].max():.5f}\tmax {metrics['max'].max():.5f}\t"
                    f"cosine {metrics['cosine'].min():.6f}\trows {metrics['rmse'].numel()}\n")


def assert_rows_close(got: torch.Tensor, want: torch.Tensor, what: str = "", bounds: Optional[dict] = None,
                      dtype: str = "bfloat16") -> None:
    bounds = bounds or BF16_BOUNDS
    assert got.shape == want.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(want.shape)}"
    assert torch.isfinite(got).all(), f"{what}: non-finite values"
    m = row_metrics(got, want)
    _note(what, dtype, m)
    bad = (m["rmse"] > bounds["rmse"]) | (m["max"] > bounds["max"]) | (m["cosine"] < bounds["cosine"])
    if bad.any():
        first = int(torch.nonzero(bad)[0, 0])
        raise AssertionError(
            f"{what}: {int(bad.sum())} of {bad.numel()} rows are off; first row {first} (row = position): relative RMSE "
            f"{m['rmse'][first]:.4f} (bound {bounds['rmse']}), relative largest difference {m['max'][first]:.4f} "
            f"(bound {bounds['max']}), cosine {m['cosine'][first]:.6f} (bound {bounds['cosine']}); worst over all rows: "
            f"{m['rmse'].max():.4f}, {m['max'].max():.4f}, {m['cosine'].min():.6f}")


def assert_close(got: torch.Tensor, want: torch.Tensor, dtype: str, what: str = "") -> None:
    if dtype == "bfloat16":
        return assert_rows_close(got, want, what)
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
