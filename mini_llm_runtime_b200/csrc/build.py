"""Compiles the native parts of the package on first use and loads them.

Every `.cu` file under `csrc/kernels/` is one kernel module and becomes one shared
library, compiled for sm_100a only; `csrc/host/*.cpp` together become the host
library (cache manager, batch planner).  A library is built when something first
asks for it, so a run compiles what its model and precision need and nothing else.
Libraries are kept under `csrc/_build/` inside the package (or, if that folder
cannot be written, under the system's temporary folder), named by a hash of their
sources and flags, so a changed source is never served by a stale build.

There is no fallback: if a library cannot be built or loaded, the caller gets a
`NativeBuildError` that says which compiler command failed and why.
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from concurrent.futures import ThreadPoolExecutor
from typing import Dict, Iterable, List, Optional

_HERE = os.path.dirname(os.path.abspath(__file__))
KERNEL_DIR = os.path.join(_HERE, "kernels")
HOST_DIR = os.path.join(_HERE, "host")

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "--shared", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"]
HOST_FLAGS = ["-O2", "-std=c++17", "-shared", "-fPIC", "-Wall"]


def cuda_home() -> str:
    for var in ("CUDA_HOME", "CUDA_PATH"):
        if os.environ.get(var):
            return os.environ[var]
    return "/usr/local/cuda"


def host_link_flags() -> List[str]:
    """The host library calls the CUDA runtime (copies, events, graph capture; linked statically like
    the kernel modules' own) and the vendor's matrix-product library."""
    home = cuda_home()
    lib = os.path.join(home, "lib64")
    return ["-I", os.path.join(home, "include"), "-L", lib, "-Wl,-rpath," + lib, "-lcublas", "-lcudart_static", "-ldl", "-lrt",
            "-lpthread"]

# Extra link flags per kernel module (none needs any today: the tensor-map encoder of the
# driver is looked up at run time through cudaGetDriverEntryPoint).
MODULE_LINK = {}

_loaded: Dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()


class NativeBuildError(RuntimeError):
    pass


def _say(message: str) -> None:
    print(f"[mini-llm-runtime_b200] {message}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    candidates = []
    for var in ("CUDA_HOME", "CUDA_PATH"):
        if os.environ.get(var):
            candidates.append(os.path.join(os.environ[var], "bin", "nvcc"))
    candidates.append("/usr/local/cuda/bin/nvcc")
    on_path = shutil.which("nvcc")
    if on_path:
        candidates.append(on_path)
    for c in candidates:
        if os.path.isfile(c) and os.access(c, os.X_OK):
            return c
    raise NativeBuildError("nvcc not found (looked in $CUDA_HOME/bin, /usr/local/cuda/bin and PATH); "
                           "the CUDA kernels of this package cannot be built")


def build_dir() -> str:
    preferred = os.path.join(_HERE, "_build")
    try:
        os.makedirs(preferred, exist_ok=True)
        probe = os.path.join(preferred, f".write_probe_{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return preferred
    except OSError:
        fallback = os.path.join(tempfile.gettempdir(), f"mini_llm_runtime_b200_build_{os.getuid()}")
        os.makedirs(fallback, exist_ok=True)
        return fallback


def _digest(paths: Iterable[str], flags: Iterable[str]) -> str:
    h = hashlib.sha256()
    for p in sorted(paths):
        h.update(os.path.basename(p).encode())
        with open(p, "rb") as f:
            h.update(f.read())
    h.update(" ".join(flags).encode())
    return h.hexdigest()[:16]


def _kernel_headers() -> List[str]:
    return [os.path.join(KERNEL_DIR, f) for f in os.listdir(KERNEL_DIR) if f.endswith((".cuh", ".h"))]


def kernel_modules() -> List[str]:
    return sorted(f[:-3] for f in os.listdir(KERNEL_DIR) if f.endswith(".cu"))


def _target(name: str):
    """(output path, command) of a library."""
    out_dir = build_dir()
    if name == "host":
        sources = sorted(os.path.join(HOST_DIR, f) for f in os.listdir(HOST_DIR) if f.endswith(".cpp"))
        link = host_link_flags()
        tag = _digest(sources, HOST_FLAGS + link)
        out = os.path.join(out_dir, f"libmlr_host-{tag}.so")
        cxx = os.environ.get("CXX") or shutil.which("g++") or shutil.which("c++")
        if not cxx:
            raise NativeBuildError("no C++ compiler found (g++ or c++) for the host library")
        return out, [cxx, *HOST_FLAGS, *sources, *link, "-o"]
    source = os.path.join(KERNEL_DIR, name + ".cu")
    if not os.path.isfile(source):
        raise NativeBuildError(f"unknown kernel module {name!r}; known: {kernel_modules()}")
    link = MODULE_LINK.get(name, [])
    tag = _digest([source, *_kernel_headers()], NVCC_FLAGS + link)
    out = os.path.join(out_dir, f"libmlr_{name}-{tag}.so")
    return out, [find_nvcc(), *NVCC_FLAGS, "-I", KERNEL_DIR, source, *link, "-o"]


def _compile(name: str, out: str, command: List[str], position: str) -> None:
    tmp = f"{out}.{os.getpid()}.{threading.get_ident()}.tmp"
    started = time.time()
    _say(f"compiling {name} {position}")
    proc = subprocess.Popen(command + [tmp], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    while True:
        try:
            output, _ = proc.communicate(timeout=15)
            break
        except subprocess.TimeoutExpired:
            _say(f"still compiling {name} ({time.time() - started:.0f} s)")
    if proc.returncode != 0:
        if os.path.exists(tmp):
            os.remove(tmp)
        raise NativeBuildError(f"building {name} failed (exit {proc.returncode}):\n  {' '.join(command)} <out>\n{output}")
    os.replace(tmp, out)
    # Older builds of the same library (other source hashes) are of no use any more.
    stem = os.path.basename(out).rsplit("-", 1)[0] + "-"
    for other in os.listdir(os.path.dirname(out)):
        if other.startswith(stem) and other.endswith(".so") and other != os.path.basename(out):
            try:
                os.remove(os.path.join(os.path.dirname(out), other))
            except OSError:
                pass
    _say(f"built {name} in {time.time() - started:.1f} s")


def ensure(names: Iterable[str]) -> None:
    """Builds the named libraries that are not built yet, several at a time."""
    todo = []
    for name in dict.fromkeys(names):
        if name in _loaded:
            continue
        out, command = _target(name)
        if not os.path.exists(out):
            todo.append((name, out, command))
    if not todo:
        return
    workers = max(1, min(len(todo), (os.cpu_count() or 2)))
    with ThreadPoolExecutor(max_workers=workers) as pool:
        futures = [pool.submit(_compile, n, o, c, f"({i + 1} of {len(todo)})") for i, (n, o, c) in enumerate(todo)]
        for f in futures:
            f.result()


def load(name: str) -> ctypes.CDLL:
    """The loaded library of a kernel module (or "host"), built first if needed."""
    with _lock:
        lib = _loaded.get(name)
        if lib is not None:
            return lib
        ensure([name])
        out, _ = _target(name)
        try:
            lib = ctypes.CDLL(out)
        except OSError as e:
            raise NativeBuildError(f"cannot load {out}: {e}") from None
        _loaded[name] = lib
        return lib


def build_all() -> List[str]:
    """Builds every library of the package; returns their paths."""
    names = ["host", *kernel_modules()]
    ensure(names)
    return [_target(n)[0] for n in names]
