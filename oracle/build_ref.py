"""Compile the reference's own runtime libraries into ``oracle/_ref/``.

TEST INFRASTRUCTURE ONLY.  The two C++ runtime libraries of the reference
build from a handful of source files with plain g++ (its compiler, which needs
LLVM/MLIR at a pinned commit and nanobind, does not).  The sources are compiled
where they lie in the reference tree; nothing is copied into this repository,
and the outputs go to ``oracle/_ref/`` (git-ignored):

* ``libcuda.so.1``                  from oracle/fake_cuda.c (a driver with no devices)
* ``libhc-cuda-runtime.so``         from gpu-runtime/cuda-runtime/src/Runtime.cpp
* ``libhc-gpu-runtime-loader.so``   from gpu-runtime/loader/src/{Loader,SharedLib}.cpp

The CMake-generated ``*_export.h`` headers are replaced by two-line stand-ins
written to ``oracle/_ref/gen/``.  Usage: ``python oracle/build_ref.py``.
"""

import os
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT = HERE / "_ref"
REFERENCE = Path(os.environ.get("HC_REFERENCE_ROOT", "/root/reference"))


def available() -> bool:
    return (REFERENCE / "gpu-runtime" / "cuda-runtime" / "src" / "Runtime.cpp").exists()


def _run(cmd):
    proc = subprocess.run([str(c) for c in cmd], capture_output=True, text=True)
    if proc.returncode:
        raise RuntimeError("reference build step failed:\n" + " ".join(map(str, cmd)) + "\n"
                           + proc.stdout + proc.stderr)


def build(force: bool = False):
    """Returns the output directory, or None when the reference tree is absent."""
    if not available():
        return None
    gen = OUT / "gen"
    gen.mkdir(parents=True, exist_ok=True)
    export = "#pragma once\n#define {0} __attribute__((visibility(\"default\")))\n"
    (gen / "hc-cuda-runtime_export.h").write_text(export.format("HC_CUDA_RUNTIME_EXPORT"))
    (gen / "hc-gpu-runtime-loader_export.h").write_text(
        export.format("HC_GPU_RUNTIME_LOADER_EXPORT"))
    cuda_inc = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda")) / "include"
    rt = REFERENCE / "gpu-runtime"
    common = ["-fPIC", "-shared", "-fvisibility=hidden", "-O1", "-w",
              "-Wl,--exclude-libs,ALL", "-Wl,-rpath,$ORIGIN"]

    fake = OUT / "libcuda.so.1"
    if force or not fake.exists():
        _run(["gcc", "-fPIC", "-shared", "-Wl,-soname,libcuda.so.1", "-o", fake,
              HERE / "fake_cuda.c"])
    backend = OUT / "libhc-cuda-runtime.so"
    if force or not backend.exists():
        _run(["g++", "-std=c++17", *common, "-include", "cstdint", "-include", "cstdio",
              "-I", gen, "-I", rt / "common" / "include", "-I", cuda_inc, "-o", backend,
              rt / "cuda-runtime" / "src" / "Runtime.cpp", fake])
    loader = OUT / "libhc-gpu-runtime-loader.so"
    if force or not loader.exists():
        _run(["g++", "-std=c++17", *common, "-include", "cstdint", "-include", "cstdio",
              "-I", gen, "-I", rt / "common" / "include", "-I", rt / "loader" / "src", "-o",
              loader, rt / "loader" / "src" / "Loader.cpp", rt / "loader" / "src" / "SharedLib.cpp",
              "-ldl"])
    return OUT


if __name__ == "__main__":
    out = build(force="--force" in sys.argv)
    print(out if out else f"reference tree not found at {REFERENCE}")
