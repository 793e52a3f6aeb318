#!/usr/bin/env python3
"""Builds the reference arm of bench.py: lilong555/mini-llm-runtime's own CUDA runtime,
compiled UNCHANGED, behind the small driver `baseline/reference_driver.cpp`.

    python baseline/build_reference.py /path/to/mini-llm-runtime        (or MLR_REFERENCE in the environment)

The reference is a CMake C++/CUDA project, not a Python package (`pip install` of its
checkout fails: neither setup.py nor pyproject.toml), and its build also wants llama.cpp
and a vendored hash library under third_party/, which the checkout does not carry.  So the
files of its CUDA runtime are copied as they are into `baseline/_ref/reference/` (the copy
travels to the GPU box; the checkout itself does not) and compiled there with nvcc for
sm_100, together with three stand-ins that live in this folder: `GgufModel` (makes a
synthetic float32 model in memory), `Tokenizer` (vocabulary size only) and
`hash/sha256/sha256.h` (a manifest field nobody reads).  The result is
`baseline/_ref/ref_bench`.  Nothing of mini-llm-runtime_b200 is compiled in.
"""
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
COPIED = ["include/minillm", "src/minillm/cuda", "src/minillm/kernels.cpp", "src/minillm/kernels_avx2.cpp",
          "src/minillm/qwen3_model.cpp"]
SOURCES = ["src/minillm/kernels.cpp", "src/minillm/kernels_avx2.cpp", "src/minillm/qwen3_model.cpp",
           "src/minillm/cuda/context.cpp", "src/minillm/cuda/matrix.cpp", "src/minillm/cuda/storage.cpp",
           "src/minillm/cuda/batch_state.cpp", "src/minillm/cuda/page_table.cpp", "src/minillm/cuda/layer.cpp",
           "src/minillm/cuda/runtime.cpp", "src/minillm/cuda/ops.cu", "src/minillm/cuda/attention.cu"]


def main() -> int:
    reference = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("MLR_REFERENCE", "")
    if not reference or not os.path.isdir(os.path.join(reference, "src", "minillm")):
        print("usage: build_reference.py /path/to/a checkout of lilong555/mini-llm-runtime (or set MLR_REFERENCE)", file=sys.stderr)
        return 2
    tree = os.path.join(OUT, "reference")
    if os.path.isdir(tree):
        shutil.rmtree(tree)
    for item in COPIED:
        source, target = os.path.join(reference, item), os.path.join(tree, item)
        os.makedirs(os.path.dirname(target), exist_ok=True)
        if os.path.isdir(source):
            shutil.copytree(source, target)
        else:
            shutil.copy2(source, target)
    nvcc = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    binary = os.path.join(OUT, "ref_bench")
    # `--pre-include cstdint`: include/minillm/cuda/matrix.h names std::uint16_t without including the
    # header that declares it, which this compiler no longer forgives; a flag, not an edit.
    command = [nvcc, "-std=c++20", "-O2", "--pre-include", "cstdint", "-gencode", "arch=compute_100,code=sm_100", "-Xcompiler", "-mavx2,-mfma,-mf16c,-pthread",
               "-I", os.path.join(tree, "include"), "-I", os.path.join(tree, "src", "minillm", "cuda"),
               "-I", os.path.join(HERE, "stand_in"), os.path.join(HERE, "reference_driver.cpp"),
               *[os.path.join(tree, s) for s in SOURCES], "-lcublas", "-o", binary]
    print(" ".join(command), flush=True)
    done = subprocess.run(command)
    if done.returncode != 0:
        return done.returncode
    print(f"built {binary}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
