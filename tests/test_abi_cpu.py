"""Host-side checks of the C-ABI libraries that need no GPU.

* every function declared in ``include/*.h`` is exported by the library that
  should export it, and every export of the reference's libraries is present;
* ``olSuggestBlockSize`` agrees with the reference implementation on a grid of
  inputs (tests/golden/reference_abi.json, recorded from the reference's own
  library by tests/golden/make_abi_golden.py);
* malformed device descriptions, garbage module images and missing backends
  fail with the reference's messages instead of crashing;
* without a driver the product path fails loudly rather than falling back.
"""

import ctypes as C
import json
import re
import subprocess
from pathlib import Path

import pytest

from hc_b200 import capi
from hc_b200.hckernel import precompiled

REPO = Path(__file__).resolve().parent.parent
NATIVE = REPO / "hc_b200" / "_native"
ABI = json.loads((REPO / "tests" / "golden" / "reference_abi.json").read_text())


def exported(lib):
    out = subprocess.run(["nm", "-D", "--defined-only", str(NATIVE / lib)], capture_output=True,
                         text=True, check=True).stdout
    return {line.split()[-1] for line in out.splitlines()}


def declared(header):
    text = (REPO / "include" / header).read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return set(re.findall(r"\b((?:olx?|hcgpu|hc|setGPU|enableFunc)[A-Za-z0-9]*)\s*\(", text))


def test_headers_match_exports():
    ol = declared("offload_api.h")
    assert len([n for n in ol if n.startswith("ol") and not n.startswith("olx")]) == 13
    assert ol <= exported("libhc-cuda-runtime.so")
    assert ol <= exported("libhc-gpu-runtime-loader.so")
    assert declared("hc_loader_api.h") == {"setGPULoaderSearchPaths", "enableFuncTracing"}
    assert declared("hc_loader_api.h") <= exported("libhc-gpu-runtime-loader.so")
    kernels = {n for n in declared("hc_b200_kernels.h") if n.startswith("hc")}
    assert len(kernels) >= 20 and kernels <= exported("libhc-b200-kernels.so")
    pyrt = {n for n in declared("hc_python_runtime.h") if n.startswith("hcgpu")}
    assert len(pyrt) == 7 and pyrt <= exported("libhc-python-runtime.so")


def test_reference_exports_are_all_present():
    assert set(ABI["backend_exports"]) <= exported("libhc-cuda-runtime.so")
    assert set(ABI["loader_exports"]) <= exported("libhc-gpu-runtime-loader.so")


def test_ctypes_prototypes_cover_the_headers():
    assert set(capi.OL_PROTOTYPES) | set(capi.OLX_PROTOTYPES) == declared("offload_api.h")
    assert set(capi.KERNELS_PROTOTYPES) == {n for n in declared("hc_b200_kernels.h")
                                            if n.startswith("hc")}
    assert set(capi.PYRUNTIME_PROTOTYPES) == {n for n in declared("hc_python_runtime.h")
                                              if n.startswith("hcgpu")}


@pytest.mark.parametrize("which", ["backend", "loader_none"])
def test_suggest_block_size_matches_reference(which):
    lib = capi.load_backend()
    for sizes, rc, expect in ABI["suggest_block_size"]:
        nd = len(sizes)
        g = (C.c_size_t * 4)(*(sizes + [8] * (4 - nd)))
        b = (C.c_size_t * 4)(9, 9, 9, 9)
        got = lib.olSuggestBlockSize(None, g, b, nd)
        assert got == rc, sizes
        assert list(b)[: len(expect)] == expect, sizes
    from hc_b200.hckernel.kernel import suggest_block_size

    for sizes, rc, expect in ABI["suggest_block_size"]:
        if rc == 0:
            assert list(suggest_block_size(sizes)) == expect


def _create(lib, desc):
    seen = []
    cb = capi.OlErrorCallback(lambda ctx, sev, text: seen.append([sev, text.decode()]))
    handle = lib.olCreateDevice(desc.encode(), cb, None)
    return handle, seen


@pytest.mark.parametrize("desc", ["cuda:x", "hip:0", "cuda", "", "cuda:"])
def test_backend_rejects_bad_descriptions_like_the_reference(desc):
    handle, seen = _create(capi.load_backend(), desc)
    assert not handle
    assert seen == ABI["backend_errors"][desc]["messages"]


@pytest.mark.parametrize("desc", ["nocolon", "foo:0", ""])
def test_loader_rejects_bad_descriptions_like_the_reference(desc):
    lib = capi.load_loader()
    lib.setGPULoaderSearchPaths(None, 0)
    handle, seen = _create(lib, desc)
    assert not handle
    # The final error is the reference's; the informational dlopen message
    # differs only in the library search text.
    assert [m for m in seen if m[0] == 0] == [m for m in ABI["loader_errors"][desc]["messages"]
                                              if m[0] == 0]


def test_loader_finds_backend_through_search_paths_and_reports_no_driver():
    import torch

    if torch.cuda.is_available():
        pytest.skip("needs a host without a CUDA driver")
    lib = capi.load_loader()
    paths = (C.c_char_p * 1)(str(NATIVE).encode())
    lib.setGPULoaderSearchPaths(paths, 1)
    handle, seen = _create(lib, "cuda:0")
    assert not handle
    assert any("CUDA driver library not found" in m for _, m in seen)


def test_no_cpu_fallback_without_driver():
    import torch

    if torch.cuda.is_available():
        pytest.skip("needs a host without a CUDA driver")
    with pytest.raises(capi.HcError, match="CUDA driver library not found"):
        capi.Context("cuda:0")
    from hc_b200._native import _dispatcher

    with pytest.raises(RuntimeError, match="cannot open device"):
        _dispatcher.Context("cuda:0")


def test_null_handles_are_rejected_not_dereferenced():
    lib = capi.load_backend()
    assert lib.olCreateModule(None, None, 0) is None
    assert lib.olGetKernel(None, b"k") is None
    assert lib.olCreateQueue(None) is None
    assert lib.olSyncQueue(None) == 1
    assert lib.olAllocDevice(None, 16, 16) is None
    g = (C.c_size_t * 3)(1, 1, 1)
    assert lib.olLaunchKernel(None, None, g, g, 3, None, 0, 0) == 1
    assert lib.olSuggestBlockSize(None, None, None, 2) == 1
    lib.olReleaseDevice(None)
    lib.olReleaseModule(None)
    lib.olReleaseKernel(None)
    lib.olReleaseQueue(None)
    lib.olDeallocDevice(None, None)
    loader = capi.load_loader()
    assert loader.olCreateModule(None, None, 0) is None
    assert loader.olLaunchKernel(None, None, g, g, 3, None, 0, 0) == 1
    loader.olReleaseQueue(None)


def test_tracing_prints_enter_and_exit(capfd):
    lib = capi.load_loader()
    lib.enableFuncTracing(1)
    try:
        _create(lib, "nocolon")
    finally:
        lib.enableFuncTracing(0)
    out = capfd.readouterr().out
    assert "olCreateDevice enter" in out and "olCreateDevice exit" in out
    _create(lib, "nocolon")
    assert "olCreateDevice" not in capfd.readouterr().out


def _elf_symbols(blob):
    """Names in the symbol table of an ELF64 image (plain header parsing)."""
    import struct

    shoff = struct.unpack_from("<Q", blob, 0x28)[0]
    shentsize, shnum = struct.unpack_from("<HH", blob, 0x3A)
    sections = [struct.unpack_from("<IIQQQQIIQQ", blob, shoff + i * shentsize) for i in range(shnum)]
    names = set()
    for s in sections:
        if s[1] != 2:  # SHT_SYMTAB
            continue
        strtab = sections[s[6]]
        for off in range(s[4], s[4] + s[5], s[9]):
            name_off = struct.unpack_from("<I", blob, off)[0]
            start = strtab[4] + name_off
            names.add(blob[start: blob.index(b"\0", start)].decode())
    return names


def test_images_are_sm100a_cubins_holding_every_listed_kernel():
    lib = capi.load_kernels()
    from hc_b200.build import KERNEL_SOURCES

    assert lib.hcImageCount() == len(KERNEL_SOURCES)
    text = (REPO / "hc_b200" / "csrc" / "launch" / "kernels_api.cpp").read_text()
    table = re.findall(r'\{"(hc_[a-z0-9_]+)", "([a-z0-9_]+)"\}', text)
    assert len(table) >= 20
    symbols = {}
    for i in range(lib.hcImageCount()):
        n = C.c_size_t(0)
        ptr = lib.hcImageData(i, C.byref(n))
        blob = C.string_at(ptr, n.value)
        assert blob[:4] == b"\x7fELF"
        # e_flags of a cubin carries the SM version in its low bits (100 -> sm_100).
        name = lib.hcImageName(i).decode()
        assert blob == (NATIVE / f"{name}.cubin").read_bytes()
        symbols[name] = _elf_symbols(blob)
    for kernel, image in table:
        if kernel.endswith("_"):
            # A prefix entry stands for a family: the gathered tile product has
            # one kernel per element type and piece shape, the element-wise
            # interpreter one per element type, packet width and input count.
            family = {s for s in symbols[image] if s.startswith(kernel)}
            expected = {
                "hc_mapped_gemm_": {f"{kernel}{t}_{sy}x{sx}" for t in ("f32", "f64")
                                    for sy in (8, 16, 32, 64) for sx in (8, 16, 32, 64)}
                | {f"{kernel}f32_128x32", f"{kernel}f32_128x64"},
                # Basic kernels for floats; extended ones (suffix x: the whole operator
                # table, validity of every element) for floats and integers.
                "hc_map_elements_": {f"{kernel}{tv}_n{n}{i}{x}"
                                     for tv, forms in (("f32_v4", ("", "x")), ("f32_v1", ("", "x")),
                                                       ("f64_v2", ("", "x")), ("f64_v1", ("", "x")),
                                                       ("i32_v4", ("x",)), ("i32_v1", ("x",)),
                                                       ("i64_v2", ("x",)), ("i64_v1", ("x",)))
                                     for n in (1, 2, 3, 4) for i in ("", "i") for x in forms},
                "hc_row_program_": {f"{kernel}{tv}_n{n}" for tv in ("f32_v4", "f32_v1", "f64_v2",
                                                                    "f64_v1")
                                    for n in (1, 2)}
                | {f"{kernel}held_{tv}_p{held}_t{threads}_n{n}" for tv in ("f32_v4", "f64_v2")
                   for held, threads in ((8, 64), (8, 96), (8, 128), (4, 256)) for n in (1, 2)},
                # One kernel per body compiled ahead of time and kernel form.
                "hc_row_fused_": {f"{kernel}{body}_{form}" for body, _, _ in precompiled.ROW_BODIES
                                  for form in ("f32_held_t64", "f32_held_t128", "f32_v4", "f32_v1",
                                               "f64_v2", "f64_v1")},
                "hc_map_fused_": {f"{kernel}{body}_{form}" for body, _, _ in precompiled.MAP_BODIES
                                  for form in ("f32_v4", "f32_v1", "f64_v2", "f64_v1")},
            }[kernel]
            assert family == expected
            for member in family:
                assert lib.hcImageName(lib.hcImageOfKernel(member.encode())).decode() == image
            continue
        assert kernel in symbols[image], (kernel, image)
        assert lib.hcImageOfKernel(kernel.encode()) >= 0
    assert lib.hcImageOfKernel(b"no_such_kernel") == -1
    assert lib.hcImageData(99, None) is None
