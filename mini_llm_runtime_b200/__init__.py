"""mini-llm-runtime_b200: a single-GPU inference engine for the dense Qwen3 decoder,
written for NVIDIA B200 (sm_100a).

    from mini_llm_runtime_b200 import LLM
    llm = LLM("/path/to/model_folder", dtype="bfloat16")
    out = llm.generate([[1, 2, 3]], max_tokens=16)

Sub-packages: `config` (typed configuration, registries), `weights` (safetensors,
loading by name, random weights), `parts` (mixer, feed-forward, norm, position
encoding, block), `cache` (pages, block tables, state slots), `engine` (the step
function, scheduler, generation), `sampling`, `ops` and `csrc` (the CUDA kernels
and native host code).
"""
from . import models as _models  # noqa: F401
from . import parts as _parts  # noqa: F401

__all__ = ["LLM", "SamplingParams"]


def __getattr__(name):
    if name in ("LLM", "SamplingParams"):
        from .engine import api
        return getattr(api, name)
    raise AttributeError(name)
