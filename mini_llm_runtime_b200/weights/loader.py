"""Binding checkpoint tensors to the tensors a model expects, by name.

Each part of a model declares the tensors it needs (`WeightSpec`: full name,
shape, role).  `load_checkpoint` opens the model folder, compares the two name
sets and every shape, and raises ONE `WeightMismatch` that lists all missing
tensors, all unexpected tensors and all wrong shapes.  The reference checks the
same things one tensor at a time (missing name: src/minillm/gguf_model.cpp:182-187;
shape: src/minillm/qwen3_model.cpp:42-49).

Stored precision is kept: bfloat16 stays bfloat16, a tensor stored in 32-bit
floats stays 32-bit, integer tables become int32; float16 (not used by this
architecture's checkpoints) is widened to float32 so that nothing is lost.
What a part does with the stored precision is its own decision at bind time.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Iterable, List, Sequence, Tuple

import torch

from .safetensors_io import SafetensorsFile, WeightFileError, open_model_files


@dataclass(frozen=True)
class WeightSpec:
    """A tensor a part needs.  `role`: "matrix" (an operand of a matrix product; it
    takes the compute precision), "vector" (norm weights and the like; they keep
    their stored precision in reduced-precision runs) or "table" (integers).
    `init` tells the random-weights mode how to fill it: ("normal", std) or
    ("one_plus_normal", std)."""
    name: str
    shape: Tuple[int, ...]
    role: str = "matrix"
    init: Tuple[str, float] = ("normal", 0.02)


class WeightMismatch(ValueError):
    """Checkpoint and model disagree; the message lists every disagreement."""

    def __init__(self, missing: List[str], unexpected: List[str], wrong: List[Tuple[str, tuple, tuple]], where: str):
        self.missing, self.unexpected, self.wrong = missing, unexpected, wrong
        lines = [f"weights in {where} do not fit the model:"]
        if missing:
            lines.append(f"  missing ({len(missing)}): " + ", ".join(missing))
        if unexpected:
            lines.append(f"  unexpected ({len(unexpected)}): " + ", ".join(unexpected))
        if wrong:
            lines.append(f"  wrong shape ({len(wrong)}): " + ", ".join(
                f"{n} is {list(got)}, expected {list(want)}" for n, got, want in wrong))
        super().__init__("\n".join(lines))


def merge_specs(specs: Iterable[WeightSpec]) -> Dict[str, WeightSpec]:
    """One spec per tensor name; a name declared twice (a tied table) must agree in shape."""
    out: Dict[str, WeightSpec] = {}
    for spec in specs:
        seen = out.get(spec.name)
        if seen is not None and tuple(seen.shape) != tuple(spec.shape):
            raise ValueError(f"tensor {spec.name!r} is declared with shapes {seen.shape} and {spec.shape}")
        out.setdefault(spec.name, spec)
    return out


def check_names_and_shapes(available: Dict[str, Tuple[int, ...]], expected: Dict[str, WeightSpec], where: str,
                           redundant: Sequence[Tuple[str, str]] = ()) -> None:
    """`redundant`: (name, twin) pairs; a stored `name` that the model does not read is not
    "unexpected" when the model reads `twin` and both have one shape."""
    allowed = {n for n, twin in redundant if twin in expected and n in available and twin in available
               and tuple(available[n]) == tuple(available[twin])}
    missing = sorted(n for n in expected if n not in available)
    unexpected = sorted(n for n in available if n not in expected and n not in allowed)
    wrong = sorted((n, tuple(available[n]), tuple(expected[n].shape)) for n in expected
                   if n in available and tuple(available[n]) != tuple(expected[n].shape))
    if missing or unexpected or wrong:
        raise WeightMismatch(missing, unexpected, wrong, where)


def _kept_precision(tensor: torch.Tensor) -> torch.Tensor:
    if tensor.dtype is torch.float16:
        return tensor.to(torch.float32)
    if tensor.dtype is torch.int64:
        return tensor.to(torch.int32)
    return tensor


def load_checkpoint(model_dir: str, expected: Dict[str, WeightSpec],
                    redundant: Sequence[Tuple[str, str]] = ()) -> Dict[str, torch.Tensor]:
    """Tensors of `model_dir` by name (CPU, mapped from the files), after the
    name and shape check.  A stored second copy named in `redundant` must equal its twin."""
    files = open_model_files(model_dir)
    owner: Dict[str, SafetensorsFile] = {}
    for f in files:
        for name in f.names():
            if name in owner:
                raise WeightFileError(f"tensor {name!r} is stored in both {owner[name].path} and {f.path}")
            owner[name] = f
    check_names_and_shapes({n: f.shape(n) for n, f in owner.items()}, expected, model_dir, redundant)
    for name, twin in redundant:
        if name in owner and name not in expected and twin in expected:
            if not torch.equal(owner[name].tensor(name), owner[twin].tensor(twin)):
                raise WeightFileError(f"{model_dir}: {name!r} is stored beside {twin!r}, which the model reads in its "
                                      f"place, but the two differ")
    return {name: _kept_precision(owner[name].tensor(name)) for name in expected}
