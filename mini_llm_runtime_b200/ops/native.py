"""Thin typed wrappers over the kernel modules' C ABI.

Each function checks that its tensors live on the GPU, are contiguous where the
kernel assumes it and have the dtype it names, passes raw pointers and the current
CUDA stream, and turns a non-zero return into `KernelError` with the module's own
message.  Nothing here computes anything and nothing falls back to another
implementation: without a GPU or without the compiled module the call raises.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from ..csrc import build

c_int, c_float, c_void_p, c_longlong = ctypes.c_int, ctypes.c_float, ctypes.c_void_p, ctypes.c_longlong
c_ulonglong, c_double = ctypes.c_ulonglong, ctypes.c_double


class KernelError(RuntimeError):
    pass


_SIGNATURES = {
    "elementwise": {
        "mlr_embed_gather": [c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p],
        "mlr_rmsnorm": [c_void_p, c_void_p, c_int, c_longlong, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int,
                        c_float, c_int, c_void_p],
        "mlr_swiglu_sliced": [c_void_p, c_int, c_longlong, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
        "mlr_qk_norm_rope_cache": [c_void_p, c_int, c_int, c_void_p, c_int, c_longlong, c_int, c_int, c_int, c_int, c_int,
                                   c_void_p, c_void_p, c_int,
                                   c_float, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                   c_void_p, c_int, c_int, c_void_p, c_void_p],
        "mlr_swiglu": [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    },
    "gemm_f32": {
        "mlr_gemm_f32": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p],
    },
    "attention_generic": {
        "mlr_attention_generic": [c_void_p, c_int, c_void_p, c_int, c_int, c_void_p, c_int, c_void_p, c_void_p,
                                  c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p, c_void_p],
    },
    "attention_bf16": {
        "mlr_attention_decode_bf16": [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p,
                                      c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int,
                                      c_void_p, c_void_p, c_void_p, c_void_p],
        "mlr_attention_decode_fresh_bf16": [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p,
                                            c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int,
                                            c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_float, c_void_p, c_int, c_void_p, c_void_p],
        "mlr_attention_prefill_bf16": [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p,
                                       c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p, c_void_p],
    },
    "attention_tcgen05": {
        "mlr_attention_prefill_tcgen05": [c_void_p, c_int, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int,
                                          c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float,
                                          c_void_p, c_void_p],
    },
    "gemm_bf16_tcgen05": {
        "mlr_gemm_bf16_tcgen05": [c_void_p, c_longlong, c_int, c_void_p, c_longlong, c_int, c_int, c_void_p, c_longlong,
                                  c_int, c_int, c_int, c_int, c_longlong, c_int, c_void_p, c_void_p],
    },
    "gemm_bf16_tcgen05_pair": {
        "mlr_gemm_bf16_tcgen05_pair": [c_void_p, c_longlong, c_int, c_void_p, c_longlong, c_int, c_int, c_void_p, c_longlong,
                                       c_int, c_void_p, c_void_p],
    },
    "sampling": {
        "mlr_sample": [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p],
    },
    "host": {
        "mlr_library_gemm": [c_void_p, c_longlong, c_int, c_void_p, c_longlong, c_int, c_int, c_void_p, c_longlong, c_int, c_int,
                             c_void_p],
    },
    "gemv_bf16": {
        "mlr_gemv_bf16": [c_void_p, c_longlong, c_int, c_int, c_void_p, c_longlong, c_int, c_void_p, c_int, c_float, c_void_p, c_int,
                          c_void_p, c_longlong, c_int, c_void_p, c_void_p],
        "mlr_gemv_bf16_fits": [c_int, c_int],
        "mlr_gemv_bf16_parts": [c_int, c_int],
        "mlr_gemv_bf16_add_prepare": [c_void_p, c_longlong, c_int, c_int, c_void_p, c_longlong, c_int, c_void_p, c_longlong, c_void_p,
                                      c_void_p, c_int, c_void_p, c_void_p, c_void_p],
        "mlr_gemv_bf16_prepared": [c_void_p, c_longlong, c_int, c_int, c_void_p, c_void_p, c_float, c_int, c_void_p, c_longlong, c_int,
                                   c_void_p, c_void_p],
    },
    "weights": {
        "mlr_normal_fill": [c_void_p, c_int, c_longlong, c_ulonglong, c_double, c_int, c_void_p],
        "mlr_finite_check": [c_void_p, c_int, c_longlong, c_void_p, c_void_p],
    },
}

_bound = {}
launch_count = 0   # kernel launches of this package since it was last reset (a measurement aid)


def register_signatures(module: str, functions: dict) -> None:
    """Lets a kernel module added later declare its functions."""
    _SIGNATURES.setdefault(module, {}).update(functions)
    _bound.pop(module, None)


def module(name: str):
    lib = _bound.get(name)
    if lib is None:
        lib = build.load(name)
        for fn, argtypes in _SIGNATURES.get(name, {}).items():
            f = getattr(lib, fn)
            f.argtypes = argtypes
            f.restype = c_int
        lib.mlr_last_error.restype = ctypes.c_char_p
        if name == "host":
            lib.mlr_exec_fail_after.argtypes = [c_longlong]
            lib.mlr_exec_fail_after.restype = None
            lib.mlr_exec_launch_count.restype = c_longlong
            lib.mlr_exec_reset_launch_count.restype = None
        _bound[name] = lib
    return lib


_functions = {}
_fail_after = None


def fail_after(launches) -> None:
    """For failure tests that must not touch the GPU's health: after `launches` more launches
    the next one fails INSTEAD of launching its kernel (None: never), whether Python makes the
    launch (`call` raises `KernelError`) or the native executor walks a program (the step
    returns its failure code).  The reference makes wrapped CUDA calls fail the same way
    (tests/cuda_runtime_tests.cpp:15-49)."""
    global _fail_after
    _fail_after = launches
    module("host").mlr_exec_fail_after(-1 if launches is None else int(launches))


def total_launches() -> int:
    """Launches of this package's kernel entry points since the last reset: those Python made and
    those the native executor made, graph replays counted with the launches they stand for."""
    return launch_count + int(module("host").mlr_exec_launch_count())


def reset_launches() -> None:
    global launch_count
    launch_count = 0
    module("host").mlr_exec_reset_launch_count()


def entry_points(module_name: str, fn: str):
    """Addresses of a kernel entry point and of its module's error text function, for ops of
    a native program."""
    lib = module(module_name)
    as_address = lambda f: ctypes.cast(f, c_void_p).value
    return as_address(getattr(lib, fn)), as_address(lib.mlr_last_error)


def is_bf16_dtype(dtype) -> int:
    if dtype is torch.bfloat16:
        return 1
    if dtype is torch.float32:
        return 0
    raise KernelError(f"kernels take float32 or bfloat16 tensors, got {dtype}")


def call(module_name: str, fn: str, *args) -> None:
    global launch_count, _fail_after
    if _fail_after is not None:
        if _fail_after <= 0:
            _fail_after = None
            raise KernelError(f"injected failure in place of {fn}")
        _fail_after -= 1
    launch_count += 1
    entry = _functions.get(fn)
    if entry is None:
        lib = module(module_name)
        entry = _functions[fn] = (getattr(lib, fn), lib)
    if entry[0](*args) != 0:
        raise KernelError(entry[1].mlr_last_error().decode("utf-8", "replace"))


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def stream() -> int:
    """The current CUDA stream's handle (of the current device).  Asked for at every launch:
    the raw query costs a fraction of a microsecond where building a Stream object costs
    several, which a step of some hundred launches feels."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def on_gpu(*tensors) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("a kernel of this package was given a tensor that is not on the GPU; "
                              "there is no CPU path")


def is_bf16(t: torch.Tensor) -> int:
    if t.dtype is torch.bfloat16:
        return 1
    if t.dtype is torch.float32:
        return 0
    raise KernelError(f"kernels take float32 or bfloat16 tensors, got {t.dtype}")


def expect(t: torch.Tensor, dtype: torch.dtype, what: str) -> None:
    if t.dtype is not dtype:
        raise KernelError(f"{what} must be {dtype}, got {t.dtype}")
    if not t.is_contiguous():
        raise KernelError(f"{what} must be contiguous")
