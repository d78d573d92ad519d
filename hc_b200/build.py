"""In-tree build of the native parts of hc_b200.

Produces, under ``hc_b200/_native/``:

* one sm_100a cubin per ``csrc/kernels/*.cu`` (``nvcc -cubin``),
* ``libhc-cuda-runtime.so``        - the ol* ABI over the CUDA driver API,
* ``libhc-gpu-runtime-loader.so``  - the backend-agnostic ol* shim,
* ``libhc-b200-kernels.so``        - the cubins (embedded) + workload launchers,
* ``libhc-python-runtime.so``      - the hcgpu* ABI (needs Python headers),
* ``_dispatcher.so``               - the pybind11 entry used by ``hckernel``.

The library names and the split follow the reference's CMake targets
(gpu-runtime/cuda-runtime/CMakeLists.txt, gpu-runtime/loader/CMakeLists.txt,
python/cpp/py-runtime/CMakeLists.txt).  Nothing here needs a GPU: nvcc
cross-compiles.  Run as ``python -m hc_b200.build`` or call :func:`build_all`.
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys
import sysconfig
from pathlib import Path

ROOT = Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
OUT = ROOT / "_native"
INCLUDE = ROOT.parent / "include"

KERNEL_SOURCES = [
    "copy2d",
    "map_elements",
    "row_program",
    "work_items",
    "map_fused",
    "row_fused",
    "softmax_rows",
    "reduce_rows",
    "reduce_all",
    "pairwise_distance",
    "mapped_gemm",
    "gemm_tiled",
    "gemm_bf16_umma",
    "gemm_f32_umma",
    "conv_f32_umma", "conv_f32_taps",
    "gemm_w8a16_umma",
    "dequant_w8",
    "selftest",
]

NVCC_FLAGS = [
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-O3",
    "-std=c++17",
]
CXX_FLAGS = [
    "-std=c++20",
    "-O2",
    "-fPIC",
    "-shared",
    "-fvisibility=hidden",
    "-Wall",
    "-Wl,-Bsymbolic",
    "-Wl,--exclude-libs,ALL",
    "-Wl,-rpath,$ORIGIN",
]


def _cuda_home() -> Path:
    for cand in (os.environ.get("CUDA_HOME"), os.environ.get("CUDA_PATH"), "/usr/local/cuda"):
        if cand and (Path(cand) / "bin" / "nvcc").exists():
            return Path(cand)
    nvcc = shutil.which("nvcc")
    if nvcc:
        return Path(nvcc).resolve().parent.parent
    raise RuntimeError("nvcc not found: set CUDA_HOME")


def _stale(target: Path, sources) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(Path(s).stat().st_mtime > t for s in sources)


def _run(cmd, verbose):
    cmd = [str(c) for c in cmd]
    if verbose:
        print("+", " ".join(cmd), flush=True)
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(
            "build step failed:\n  " + " ".join(cmd) + "\n" + proc.stdout + proc.stderr
        )
    if verbose and (proc.stdout or proc.stderr):
        print(proc.stdout + proc.stderr, flush=True)


def build_cubins(verbose=False, force=False):
    """Compile every kernel source to an sm_100a cubin."""
    cuda = _cuda_home()
    OUT.mkdir(exist_ok=True)
    headers = [*(CSRC / "kernels").glob("*.cuh"), *(CSRC / "kernels").glob("*.h")]
    outs = []
    for name in KERNEL_SOURCES:
        src = CSRC / "kernels" / f"{name}.cu"
        out = OUT / f"{name}.cubin"
        if force or _stale(out, [src, *headers]):
            _run([cuda / "bin" / "nvcc", *NVCC_FLAGS, "-cubin", "-o", out, src], verbose)
        outs.append(out)
    return outs


# Kernel sources embedded as text: what a run-time specialisation compiles
# (csrc/launch/specialise.cpp).
EMBEDDED_SOURCES = ["map_fused.cu", "row_fused.cu", "work_items.cu", "fused_machine.cuh",
                    "map_machine.cuh", "map_params.h", "items_params.h"]


def _write_images_asm(cubins, path: Path):
    """Assembly that embeds each cubin and a name/begin/end table, and the same
    for the kernel sources of EMBEDDED_SOURCES.  The files are named by file
    name only; the assembler finds them through ``-I``."""
    lines = ['.section .rodata', '.balign 16']
    for i, name in enumerate(EMBEDDED_SOURCES):
        lines += [
            f"hc_src_name_{i}: .asciz \"{name}\"",
            ".balign 16",
            f"hc_src_begin_{i}: .incbin \"{name}\"",
            f"hc_src_end_{i}: .byte 0",
            ".balign 16",
        ]
    for i, c in enumerate(cubins):
        lines += [
            f"hc_img_name_{i}: .asciz \"{c.stem}\"",
            ".balign 16",
            f"hc_img_begin_{i}: .incbin \"{c.name}\"",
            f"hc_img_end_{i}:",
            ".balign 16",
        ]
    # The table holds addresses, so it lives in a relocatable read-only section.
    lines += ['.section .data.rel.ro,"aw"', ".globl hc_b200_images", ".balign 8",
              "hc_b200_images:"]
    for i in range(len(cubins)):
        lines += [f"  .quad hc_img_name_{i}", f"  .quad hc_img_begin_{i}", f"  .quad hc_img_end_{i}"]
    lines += [".globl hc_b200_sources", ".balign 8", "hc_b200_sources:"]
    for i in range(len(EMBEDDED_SOURCES)):
        lines += [f"  .quad hc_src_name_{i}", f"  .quad hc_src_begin_{i}", f"  .quad hc_src_end_{i}"]
    lines += [
        ".section .rodata",
        ".globl hc_b200_source_count",
        ".balign 4",
        "hc_b200_source_count:",
        f"  .long {len(EMBEDDED_SOURCES)}",
        ".globl hc_b200_image_count",
        ".balign 4",
        "hc_b200_image_count:",
        f"  .long {len(cubins)}",
        '.section .note.GNU-stack,"",@progbits',
    ]
    path.write_text("\n".join(lines) + "\n")


def build_libs(verbose=False, force=False):
    cuda = _cuda_home()
    cxx = os.environ.get("CXX", "g++")
    inc = ["-I", INCLUDE, "-I", cuda / "include"]
    cubins = build_cubins(verbose, force)

    backend = OUT / "libhc-cuda-runtime.so"
    srcs = [CSRC / "runtime" / "cuda_runtime.cpp", CSRC / "runtime" / "driver_api.hpp",
            INCLUDE / "offload_api.h"]
    if force or _stale(backend, srcs):
        _run([cxx, *CXX_FLAGS, *inc, "-o", backend, srcs[0], "-ldl"], verbose)

    loader = OUT / "libhc-gpu-runtime-loader.so"
    srcs = [CSRC / "loader" / "loader.cpp", INCLUDE / "offload_api.h"]
    if force or _stale(loader, srcs):
        _run([cxx, *CXX_FLAGS, *inc, "-o", loader, srcs[0], "-ldl"], verbose)

    kernels = OUT / "libhc-b200-kernels.so"
    host_src = CSRC / "launch" / "host_api.cpp"
    spec_src = CSRC / "launch" / "specialise.cpp"
    srcs = [CSRC / "launch" / "kernels_api.cpp", host_src, spec_src,
            CSRC / "launch" / "context.hpp",
            *(CSRC / "kernels" / name for name in EMBEDDED_SOURCES),
            INCLUDE / "hc_b200_kernels.h",
            INCLUDE / "offload_api.h", CSRC / "kernels" / "mapped_params.h",
            CSRC / "kernels" / "map_params.h", CSRC / "kernels" / "fused_programs.h",
            CSRC / "kernels" / "items_params.h", CSRC / "kernels" / "conv_params.h", loader,
            *cubins]
    static_src = CSRC / "launch" / "w8a16_static.cu"
    srcs.append(static_src)
    if force or _stale(kernels, srcs):
        asm = OUT / "images_gen.S"
        _write_images_asm(cubins, asm)
        # The one translation unit that uses the CUDA runtime API (it owns a
        # __device__ array and needs cudaGetSymbolAddress): host + device code
        # in one object, CUDA runtime linked statically.
        static_obj = OUT / "w8a16_static.o"
        _run([cuda / "bin" / "nvcc", *NVCC_FLAGS, "-Xcompiler", "-fPIC,-fvisibility=hidden",
              "-cudart", "static", *inc, "-c", "-o", static_obj, static_src], verbose)
        _run([cxx, *CXX_FLAGS, *inc, "-I", OUT, "-I", CSRC / "kernels", "-o", kernels, srcs[0],
              host_src, spec_src, asm, static_obj,
              "-L", OUT, "-lhc-gpu-runtime-loader", "-L", cuda / "lib64", "-lcudart_static",
              "-lrt", "-lpthread", "-ldl"], verbose)

    pyinc = sysconfig.get_paths()["include"]
    have_python_headers = (Path(pyinc) / "Python.h").exists()
    built = [backend, loader, kernels]
    if have_python_headers:
        import pybind11

        pyflags = ["-I", pyinc, "-I", pybind11.get_include()]
        pyrt = OUT / "libhc-python-runtime.so"
        srcs = [CSRC / "pyruntime" / "py_runtime.cpp", CSRC / "pyruntime" / "array_arg.hpp",
                INCLUDE / "hc_python_runtime.h", loader]
        if all(Path(s).exists() for s in srcs) and (force or _stale(pyrt, srcs)):
            _run([cxx, *CXX_FLAGS, *inc, *pyflags, "-o", pyrt, srcs[0],
                  "-L", OUT, "-lhc-gpu-runtime-loader", "-ldl"], verbose)
        if pyrt.exists():
            built.append(pyrt)
        disp = OUT / "_dispatcher.so"
        srcs = [CSRC / "dispatch" / "dispatcher.cpp", CSRC / "pyruntime" / "array_arg.hpp",
                INCLUDE / "hc_b200_kernels.h", kernels]
        if all(Path(s).exists() for s in srcs) and (force or _stale(disp, srcs)):
            _run([cxx, *CXX_FLAGS, *inc, *pyflags, "-I", CSRC / "pyruntime", "-o", disp, srcs[0],
                  "-L", OUT, "-lhc-b200-kernels", "-lhc-gpu-runtime-loader", "-ldl"], verbose)
        if disp.exists():
            built.append(disp)
    return built


def build_all(verbose=False, force=False):
    """Build everything; returns the list of shared libraries produced."""
    return build_libs(verbose, force)


if __name__ == "__main__":
    libs = build_all(verbose="-q" not in sys.argv, force="--force" in sys.argv)
    for lib in libs:
        print(lib)
