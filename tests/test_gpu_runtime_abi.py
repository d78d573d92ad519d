"""The ol* and hcgpu* C-ABIs on a real GPU, used the way the reference's JIT'd
host code uses them (mlir/lib/Transforms/GpuToGpuRuntime.cpp:163-350;
python/cpp/py-runtime/src/GpuRuntime.cpp:26-69): create a device and a queue,
build a module from a binary blob, fetch a kernel, pack ``void *args[]``,
launch, synchronise - through the loader, through the backend directly, and
through the py-runtime - plus the host-side failure paths of each call.
"""

import ctypes as C

import numpy as np
import pytest
import torch

from hc_b200 import capi

pytestmark = pytest.mark.gpu


def _image(name=b"hc_copy2d"):
    k = capi.load_kernels()
    n = C.c_size_t(0)
    ptr = k.hcImageData(k.hcImageOfKernel(name), C.byref(n))
    return ptr, n.value


def _copy_args(src, dst, rows, cols):
    """args[] of hc_copy2d: (src, dst, rows, rowBytes, srcPitch, dstPitch, packet)."""
    vals = [C.c_void_p(src), C.c_void_p(dst), C.c_longlong(rows), C.c_longlong(cols * 4),
            C.c_longlong(cols * 4), C.c_longlong(cols * 4), C.c_int(4)]
    return vals, (C.c_void_p * 7)(*[C.addressof(v) for v in vals])


@pytest.mark.parametrize("which", ["loader", "backend"])
def test_ol_lifecycle_alloc_copy_launch(which):
    lib = capi.load_loader() if which == "loader" else capi.load_backend()
    if which == "loader":
        paths = (C.c_char_p * 1)(str(capi.NATIVE_DIR).encode())
        lib.setGPULoaderSearchPaths(paths, 1)
    seen = []
    cb = capi.OlErrorCallback(lambda ctx, sev, text: seen.append((sev, text.decode())))
    dev = lib.olCreateDevice(b"cuda:0", cb, None)
    assert dev, seen
    q = lib.olCreateQueue(dev)
    assert q, seen
    assert lib.olxQueueNativeHandle(q)
    sms = C.c_longlong(0)
    assert lib.olxDeviceAttribute(dev, capi.OLX_DEVICE_SM_COUNT, C.byref(sms)) == 0
    assert sms.value > 0

    ptr, n = _image()
    mod = lib.olCreateModule(dev, ptr, n)
    assert mod, seen
    k = lib.olGetKernel(mod, b"hc_copy2d")
    assert k, seen

    rows, cols = 37, 53
    host = np.arange(rows * cols, dtype=np.int32)
    back = np.zeros_like(host)
    nbytes = host.nbytes
    d_src = lib.olAllocDevice(q, nbytes, 256)
    d_dst = lib.olAllocDevice(q, nbytes, 4096)  # over-aligned on purpose
    assert d_src and d_dst and d_dst % 4096 == 0
    assert lib.olxMemcpyHtoD(q, d_src, host.ctypes.data, nbytes) == 0
    assert lib.olxMemsetD8(q, d_dst, 0, nbytes) == 0

    g = (C.c_size_t * 3)(rows, 1, 1)
    blk = (C.c_size_t * 3)(9, 9, 9)
    assert lib.olSuggestBlockSize(k, g, blk, 3) == 0 and list(blk) == [rows, 1, 1]
    keep, args = _copy_args(d_src, d_dst, rows, cols)
    grid = (C.c_size_t * 3)(1, 8, 1)
    block = (C.c_size_t * 3)(256, 1, 1)
    assert lib.olLaunchKernel(q, k, grid, block, 3, args, 7, 0) == 0, seen
    assert lib.olxMemcpyDtoH(q, back.ctypes.data, d_dst, nbytes) == 0
    assert lib.olSyncQueue(q) == 0
    assert np.array_equal(back, host)

    # Failure paths: each returns an error and reports through the callback.
    seen.clear()
    assert lib.olLaunchKernel(q, k, grid, block, 2, args, 7, 0) == 1
    assert seen[-1] == (0, "Invalid launch dims: 2")
    assert not lib.olGetKernel(mod, b"no_such_kernel")
    assert "cuModuleGetFunction" in seen[-1][1] and "CUDA_ERROR_NOT_FOUND" in seen[-1][1]
    garbage = (C.c_ubyte * 64)(*([0x5A] * 64))
    assert not lib.olCreateModule(dev, garbage, 64)
    assert "Invalid module image" in seen[-1][1]
    truncated = C.string_at(ptr, 200)  # ELF header present, sections cut off
    buf = C.create_string_buffer(truncated, 200)
    assert not lib.olCreateModule(dev, buf, 200)
    assert "truncated ELF" in seen[-1][1]
    assert not lib.olAllocDevice(q, 16, 3)  # alignment must be a power of two
    assert lib.olLaunchKernel(q, k, grid, block, 3, args, 7, 10 << 20) == 1  # 10 MiB of smem
    assert "cuFuncSetAttribute" in seen[-1][1] or "cuLaunchKernel" in seen[-1][1]
    assert lib.olSyncQueue(q) == 0  # the context survived all of it

    lib.olDeallocDevice(q, d_src)
    lib.olDeallocDevice(q, d_dst)
    lib.olReleaseKernel(k)
    lib.olReleaseModule(mod)
    lib.olReleaseQueue(q)
    lib.olReleaseDevice(dev)


def test_loader_tracing_shows_launch_geometry(capfd):
    lib = capi.load_loader()
    paths = (C.c_char_p * 1)(str(capi.NATIVE_DIR).encode())
    lib.setGPULoaderSearchPaths(paths, 1)
    dev = lib.olCreateDevice(b"cuda:0", capi.OlErrorCallback(lambda *a: None), None)
    q = lib.olCreateQueue(dev)
    ptr, n = _image()
    mod = lib.olCreateModule(dev, ptr, n)
    k = lib.olGetKernel(mod, b"hc_copy2d")
    src = torch.arange(64, dtype=torch.int32, device="cuda")
    dst = torch.zeros_like(src)
    torch.cuda.synchronize()
    keep, args = _copy_args(src.data_ptr(), dst.data_ptr(), 4, 16)
    grid, block = (C.c_size_t * 3)(1, 4, 1), (C.c_size_t * 3)(256, 1, 1)
    lib.enableFuncTracing(1)
    try:
        assert lib.olLaunchKernel(q, k, grid, block, 3, args, 7, 0) == 0
        assert lib.olSyncQueue(q) == 0
    finally:
        lib.enableFuncTracing(0)
    out = capfd.readouterr().out
    assert "olLaunchKernel grid: [1, 4, 1], blocks [256, 1, 1], nargs 7, shMem 0" in out
    assert "olLaunchKernel exit" in out and "olSyncQueue enter" in out
    assert torch.equal(dst, src)
    lib.olReleaseKernel(k)
    lib.olReleaseModule(mod)
    lib.olReleaseQueue(q)
    lib.olReleaseDevice(dev)


def test_hcgpu_get_kernel_and_launch_like_jit_host_code():
    rt = capi.load_python_runtime()
    rt.hcgpuSetRuntimeSearchPaths([str(capi.NATIVE_DIR).encode()])
    ptr, n = _image()
    handle = C.c_void_p(0)  # the per-call-site cache slot the JIT emits
    k = rt.hcgpuGetKernel(C.byref(handle), b"cuda:0", ptr, n, b"hc_copy2d")
    assert k and handle.value == k
    assert rt.hcgpuGetKernel(C.byref(handle), b"cuda:0", ptr, n, b"hc_copy2d") == k  # cached

    src = torch.arange(111 * 813, dtype=torch.int32, device="cuda").reshape(111, 813)
    dst = torch.zeros_like(src)
    torch.cuda.synchronize()

    class Desc(C.Structure):
        _fields_ = [("allocated", C.c_void_p), ("aligned", C.c_void_p), ("offset", C.c_ssize_t),
                    ("sizes", C.c_ssize_t * 2), ("strides", C.c_ssize_t * 2)]

    ds, dd = Desc(), Desc()
    assert rt.hcgpuConvertPyArray(None, src, 2, C.byref(ds)) == 0
    assert rt.hcgpuConvertPyArray(None, dst, 2, C.byref(dd)) == 0
    assert ds.aligned == src.data_ptr() and list(ds.sizes) == [111, 813]

    g = (C.c_size_t * 3)(813, 111, 1)  # x is the last work dimension
    blk = (C.c_size_t * 3)()
    rt.hcgpuSuggestBlockSize(k, g, blk, 3)
    assert list(blk) == [813, 1, 1]
    keep, args = _copy_args(ds.aligned, dd.aligned, ds.sizes[0], ds.sizes[1])
    grid, block = (C.c_size_t * 3)(4, 111, 1), (C.c_size_t * 3)(256, 1, 1)
    rt.hcgpuLaunchKernel(k, grid, block, 3, args, 7, 0)  # returns after the kernel finished
    assert torch.equal(dst, src)


@pytest.mark.parametrize("which", ["loader", "backend"])
def test_tensor_map_encoders_accept_and_refuse(which):
    """olxEncodeTensorMap2D / olxEncodeTensorMapTiled: descriptors of rank 2 to 5 for
    aligned tensors; a bad rank, a pitch that is not a multiple of 16 bytes, a box
    wider than the swizzle span and an unaligned base are refused with a message."""
    lib = capi.load_loader() if which == "loader" else capi.load_backend()
    if which == "loader":
        paths = (C.c_char_p * 1)(str(capi.NATIVE_DIR).encode())
        lib.setGPULoaderSearchPaths(paths, 1)
    seen = []
    cb = capi.OlErrorCallback(lambda ctx, sev, text: seen.append((sev, text.decode())))
    dev = lib.olCreateDevice(b"cuda:0", cb, None)
    assert dev, seen
    q = lib.olCreateQueue(dev)
    base = lib.olAllocDevice(q, 1 << 20, 1024)
    raw = C.create_string_buffer(128 + 64)
    desc = C.c_void_p((C.addressof(raw) + 63) & ~63)  # 64-byte aligned, 128 bytes

    def tiled(rank, dims, pitches, box, swizzle=128, at=base):
        return lib.olxEncodeTensorMapTiled(dev, desc, 1, at, rank, (C.c_size_t * len(dims))(*dims),
                                           (C.c_size_t * max(1, len(pitches)))(*pitches),
                                           (C.c_uint * len(box))(*box), swizzle)

    assert lib.olxEncodeTensorMap2D(dev, desc, 1, base, 64, 128, 512, 16, 32, 128) == 0, seen
    # [N = 2][H * W = 400][C = 64] floats, a box of 32 channels x 136 positions.
    assert tiled(3, [64, 400, 2], [256, 400 * 256], [32, 136, 1]) == 0, seen
    # [N = 2][H = 20][W = 20][C = 64], a box of 32 channels x 64 x 2 pixels.
    assert tiled(4, [64, 20, 20, 2], [256, 20 * 256, 400 * 256], [32, 16, 8, 1]) == 0, seen
    assert tiled(5, [64, 5, 4, 20, 2], [256, 5 * 256, 20 * 256, 400 * 256], [32, 2, 2, 4, 1]) == 0
    seen.clear()
    assert tiled(6, [64] * 6, [256] * 5, [32] * 6) == 1
    assert "Invalid tensor map geometry" in seen[-1][1]
    assert tiled(3, [64, 400, 2], [250, 400 * 256], [32, 136, 1]) == 1   # pitch % 16 != 0
    assert tiled(3, [64, 400, 2], [256, 400 * 256], [64, 136, 1]) == 1   # 256-byte box, swizzle 128
    assert tiled(3, [64, 400, 2], [256, 400 * 256], [32, 300, 1]) == 1   # a box dimension > 256
    assert tiled(3, [64, 400, 2], [256, 400 * 256], [32, 136, 1], at=base + 4) == 1
    assert all("Invalid tensor map geometry" in text for _, text in seen)
    lib.olDeallocDevice(q, base)
    lib.olReleaseQueue(q)
    lib.olReleaseDevice(dev)
