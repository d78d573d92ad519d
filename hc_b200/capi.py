"""ctypes bindings of the C-ABI libraries in ``hc_b200/_native``.

This module only declares prototypes and loads the libraries; it holds no
logic of its own.  It is what a foreign-language host would write against
``include/*.h``, and the GPU parity tests call the kernels through it so that
they exercise the C-ABI itself.

The libraries are never built implicitly.  If one is missing the import fails
with an error that names the build command: there is no CPU fallback.
"""

from __future__ import annotations

import ctypes as C
from pathlib import Path

NATIVE_DIR = Path(__file__).resolve().parent / "_native"

OlErrorCallback = C.CFUNCTYPE(None, C.c_void_p, C.c_int, C.c_char_p)

# hc_b200_kernels.h: enum HcDType
HC_F32, HC_F64, HC_BF16, HC_I8, HC_I32, HC_I64 = 0, 1, 2, 3, 4, 5

# offload_api.h: OLX_DEVICE_*
OLX_DEVICE_SM_COUNT = 1
OLX_DEVICE_CC_MAJOR = 2
OLX_DEVICE_CC_MINOR = 3
OLX_DEVICE_L2_BYTES = 4
OLX_DEVICE_MAX_SMEM_OPTIN = 5
OLX_DEVICE_ORDINAL = 6

_sz = C.c_size_t
_vp = C.c_void_p
_ll = C.c_longlong



class HcMappedOperand(C.Structure):
    """include/hc_b200_kernels.h: one array of hcMappedGemm with its tables."""

    _fields_ = [
        ("base", _vp),
        ("map", _vp),
        ("lin", _vp),
        ("origins", _vp),
        ("shape", C.c_int * 4),
        ("stride", _ll * 4),
        ("lo", C.c_int * 4),
        ("hi", C.c_int * 4),
        ("transposed", C.c_int),
        ("sharedRun", C.c_int),
    ]


class HcMapProgram(C.Structure):
    """include/hc_b200_kernels.h: the arrays and the program of hcMapElements."""

    _fields_ = [
        ("inputs", _vp * 4),
        ("inPitch", _ll * 4),
        ("out", _vp),
        ("outPitch", _ll),
        ("rows", _ll),
        ("cols", _ll),
        ("nInputs", C.c_int),
        ("nInstr", C.c_int),
        ("code", C.c_uint * 32),
        ("consts", C.c_double * 8),
    ]


class HcPeerOutputs(C.Structure):
    """include/hc_b200_kernels.h: where a rank's rows go in every rank's buffer."""

    _fields_ = [("base", _vp * 8), ("count", C.c_int)]


class HcItemProgram(C.Structure):
    """include/hc_b200_kernels.h: the arrays and the program of hcWorkItems."""

    _fields_ = [
        ("inputs", _vp * 4),
        ("inPitch", _ll * 4),
        ("inRow", C.c_int * 4),
        ("inCol", C.c_int * 4),
        ("out", _vp),
        ("outPitch", _ll),
        ("rows", _ll),
        ("cols", _ll),
        ("groupRows", C.c_int),
        ("groupCols", C.c_int),
        ("nInputs", C.c_int),
        ("nInstr", C.c_int),
        ("code", C.c_uint * 48),
        ("consts", C.c_double * 8),
        ("guardLo", (_ll * 2) * 2),
        ("guardHi", (_ll * 2) * 2),
        ("tileScale", (C.c_int * 2) * 4),
        ("tileOffset", (C.c_int * 2) * 4),
        ("tileMod", (C.c_int * 2) * 4),
        ("tileFill", C.c_double),
    ]


# name -> (restype, argtypes), exactly as declared in include/offload_api.h
OL_PROTOTYPES = {
    "olCreateDevice": (_vp, [C.c_char_p, OlErrorCallback, _vp]),
    "olReleaseDevice": (None, [_vp]),
    "olCreateModule": (_vp, [_vp, _vp, _sz]),
    "olReleaseModule": (None, [_vp]),
    "olGetKernel": (_vp, [_vp, C.c_char_p]),
    "olReleaseKernel": (None, [_vp]),
    "olSuggestBlockSize": (C.c_int, [_vp, C.POINTER(_sz), C.POINTER(_sz), _sz]),
    "olCreateQueue": (_vp, [_vp]),
    "olReleaseQueue": (None, [_vp]),
    "olSyncQueue": (C.c_int, [_vp]),
    "olAllocDevice": (_vp, [_vp, _sz, _sz]),
    "olDeallocDevice": (None, [_vp, _vp]),
    "olLaunchKernel": (
        C.c_int,
        [_vp, _vp, C.POINTER(_sz), C.POINTER(_sz), _sz, C.POINTER(_vp), _sz, _sz],
    ),
}
OLX_PROTOTYPES = {
    "olxQueueNativeHandle": (_vp, [_vp]),
    "olxMemcpyHtoD": (C.c_int, [_vp, _vp, _vp, _sz]),
    "olxMemcpyDtoH": (C.c_int, [_vp, _vp, _vp, _sz]),
    "olxMemsetD8": (C.c_int, [_vp, _vp, C.c_int, _sz]),
    "olxDeviceAttribute": (C.c_int, [_vp, C.c_int, C.POINTER(_ll)]),
    "olxEncodeTensorMap2D": (
        C.c_int,
        [_vp, _vp, C.c_int, _vp, _sz, _sz, _sz, C.c_uint, C.c_uint, C.c_int],
    ),
    "olxEncodeTensorMapTiled": (
        C.c_int,
        [_vp, _vp, C.c_int, _vp, C.c_int, C.POINTER(_sz), C.POINTER(_sz), C.POINTER(C.c_uint),
         C.c_int],
    ),
    "olxMaxActiveClusters": (
        C.c_int,
        [_vp, _vp, C.c_uint, _sz, C.c_uint, C.POINTER(C.c_int)],
    ),
    "olxDeviceContextEnter": (C.c_int, [_vp]),
    "olxDeviceContextLeave": (C.c_int, [_vp]),
    "olxPointerDevice": (C.c_int, [_vp, _vp, C.POINTER(C.c_int)]),
    "olxCreateEvent": (_vp, [_vp, C.c_int]),
    "olxReleaseEvent": (None, [_vp, _vp]),
    "olxRecordEvent": (C.c_int, [_vp, _vp]),
    "olxQueueWaitEvent": (C.c_int, [_vp, _vp]),
    "olxEventElapsedMs": (C.c_int, [_vp, _vp, _vp, C.POINTER(C.c_float)]),
    "olxHostRegister": (C.c_int, [_vp, _vp, _sz]),
    "olxHostUnregister": (C.c_int, [_vp, _vp]),
}
LOADER_EXTRA_PROTOTYPES = {
    "setGPULoaderSearchPaths": (None, [C.POINTER(C.c_char_p), _sz]),
    "enableFuncTracing": (None, [C.c_int]),
}
# include/hc_b200_kernels.h
KERNELS_PROTOTYPES = {
    "hcImageCount": (C.c_int, []),
    "hcImageName": (C.c_char_p, [C.c_int]),
    "hcImageData": (_vp, [C.c_int, C.POINTER(_sz)]),
    "hcImageOfKernel": (C.c_int, [C.c_char_p]),
    "hcCreateContext": (_vp, [C.c_char_p, OlErrorCallback, _vp]),
    "hcReleaseContext": (None, [_vp]),
    "hcContextDevice": (_vp, [_vp]),
    "hcContextQueue": (_vp, [_vp]),
    "hcContextStream": (_vp, [_vp]),
    "hcSynchronize": (C.c_int, [_vp]),
    "hcLastError": (C.c_char_p, [_vp]),
    "hcLaunchCount": (_ll, [_vp]),
    "hcKernelStatus": (C.c_int, [_vp, C.POINTER(C.c_int)]),
    "hcSetOption": (C.c_int, [_vp, C.c_char_p, _ll]),
    "hcSpecialisedPrograms": (_ll, [_vp, C.c_int]),
    "hcSpecialiseNote": (C.c_char_p, [_vp]),
    "hcSpecialiseCompile": (
        _ll, [C.POINTER(HcMapProgram), C.c_int, C.c_int, C.c_int, C.c_int, _vp, _sz, C.c_char_p,
              _sz]
    ),
    "hcSpecialiseCompileItems": (
        _ll, [C.POINTER(C.c_uint32), C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, _vp, _sz,
              C.c_char_p, _sz]
    ),
    "hcSelfTestWaitTimeout": (
        C.c_int,
        [_vp, C.c_ulonglong, C.POINTER(C.c_int), C.POINTER(C.c_ulonglong), C.POINTER(C.c_int)],
    ),
    "hcCopy2D": (C.c_int, [_vp, _vp, _vp, _ll, _ll, _ll, _ll, C.c_int]),
    "hcSoftmaxRows": (C.c_int, [_vp, _vp, _vp, _ll, _ll, _ll, _ll, C.c_int]),
    "hcReduceRows": (C.c_int, [_vp, _vp, _vp, _vp, _ll, _ll, _ll, C.c_int]),
    "hcReduceAll": (C.c_int, [_vp, _vp, _ll, _vp, C.c_int, C.c_int]),
    "hcSoftmaxRowsPeers": (
        C.c_int, [_vp, _vp, C.POINTER(HcPeerOutputs), _ll, _ll, _ll, _ll, C.c_int]
    ),
    "hcGemmBf16Peers": (
        C.c_int, [_vp, _vp, _vp, C.POINTER(HcPeerOutputs), _ll, _ll, _ll, _ll, _ll, _ll]
    ),
    "hcGemmW8A16Peers": (
        C.c_int, [_vp, _vp, _vp, _vp, C.POINTER(HcPeerOutputs), _vp, _sz, _ll, _ll, _ll, _ll,
                  _ll, _ll]
    ),
    "hcReduceRowsPeers": (
        C.c_int, [_vp, _vp, C.POINTER(HcPeerOutputs), _ll, _ll, _ll, _ll, C.c_int]
    ),
    "hcPairwiseDistance": (
        C.c_int, [_vp, _vp, _vp, _vp, _ll, _ll, _ll, _ll, _ll, _ll, C.c_int]
    ),
    "hcMapElements": (C.c_int, [_vp, C.POINTER(HcMapProgram), C.c_int]),
    "hcRowProgram": (C.c_int, [_vp, C.POINTER(HcMapProgram), C.c_int]),
    "hcWorkItems": (C.c_int, [_vp, C.POINTER(HcItemProgram), C.c_int]),
    "hcMappedGemm": (
        C.c_int,
        [_vp, C.POINTER(HcMappedOperand), C.POINTER(HcMappedOperand),
         C.POINTER(HcMappedOperand), _ll, C.c_int, C.c_int, C.c_int, C.c_int],
    ),
    "hcGemmTiled": (C.c_int, [_vp, _vp, _vp, _vp, _ll, _ll, _ll, _ll, _ll, _ll, C.c_int]),
    "hcGemmBf16": (C.c_int, [_vp, _vp, _vp, _vp, _ll, _ll, _ll, _ll, _ll, _ll]),
    "hcGemmF32TensorWorkspaceBytes": (_sz, [_ll, _ll, _ll]),
    "hcGemmF32Tensor": (
        C.c_int, [_vp, _vp, _vp, _vp, _vp, _sz, _ll, _ll, _ll, _ll, _ll, _ll]
    ),
    "hcConvF32TensorWorkspaceBytes": (_sz, [_ll, _ll, _ll, _ll, _ll, _ll, _ll]),
    "hcConvF32Tensor": (
        C.c_int, [_vp, _vp, _vp, _vp, _ll, _ll, _ll, _ll, _ll, _ll, _ll, _ll, _vp, _sz]
    ),
    "hcGemmW8A16WorkspaceBytes": (_sz, [_ll, _ll]),
    "hcGemmW8A16BandedBytes": (_sz, [_ll, _ll]),
    "hcGemmW8A16": (
        C.c_int,
        [_vp, _vp, _vp, _vp, _vp, _vp, _sz, _ll, _ll, _ll, _ll, _ll, _ll],
    ),
    "hcDequantW8": (C.c_int, [_vp, _vp, _vp, _ll, _ll, _ll, _ll]),
    "hcGemmW8A16StaticMaxBytes": (_sz, []),
    "hcGemmW8A16Static": (C.c_int, [_vp, _vp, _vp, _vp, _vp, _ll, _ll, _ll, _ll, _ll, _ll]),
    "hcReportError": (C.c_int, [_vp, C.c_char_p]),
    "hcHostPin": (C.c_int, [_vp, _vp, _sz]),
    "hcHostUnpin": (C.c_int, [_vp, _vp]),
    "hcSoftmaxRowsHost": (C.c_int, [_vp, _vp, _vp, _ll, _ll, _ll, _ll, C.c_int]),
    "hcReduceRowsHost": (C.c_int, [_vp, _vp, _vp, _vp, _ll, _ll, _ll, C.c_int]),
    "hcGemmBf16Host": (C.c_int, [_vp, _vp, _vp, _vp, _ll, _ll, _ll, _ll, _ll, _ll]),
}
# include/hc_python_runtime.h
PYRUNTIME_PROTOTYPES = {
    "hcgpuEnableTraceFunctions": (None, [C.c_int]),
    "hcgpuSetRuntimeSearchPaths": (None, [C.py_object]),
    "hcgpuConvertPyArray": (C.c_int, [_vp, C.py_object, C.c_int, _vp]),
    "hcgpuConvertPyInt64": (C.c_int, [_vp, C.py_object, C.POINTER(C.c_int64)]),
    "hcgpuGetKernel": (_vp, [C.POINTER(_vp), C.c_char_p, _vp, _sz, C.c_char_p]),
    "hcgpuSuggestBlockSize": (None, [_vp, C.POINTER(_sz), C.POINTER(_sz), _sz]),
    "hcgpuLaunchKernel": (
        None,
        [_vp, C.POINTER(_sz), C.POINTER(_sz), _sz, C.POINTER(_vp), _sz, _sz],
    ),
}


def _declare(lib, table):
    for name, (restype, argtypes) in table.items():
        fn = getattr(lib, name)
        fn.restype = restype
        fn.argtypes = argtypes
    return lib


def _open(name: str, loader=C.CDLL):
    path = NATIVE_DIR / name
    if not path.exists():
        raise ImportError(
            f"{path} is missing: build the native libraries first "
            f"(`python -m hc_b200.build`); hc_b200 has no CPU fallback"
        )
    return loader(str(path))


def load_backend():
    """libhc-cuda-runtime.so (the 13 ol* + the olx* additions)."""
    return _declare(_declare(_open("libhc-cuda-runtime.so"), OL_PROTOTYPES), OLX_PROTOTYPES)


def load_loader():
    """libhc-gpu-runtime-loader.so (same ABI + the two loader-only exports)."""
    lib = _declare(_declare(_open("libhc-gpu-runtime-loader.so"), OL_PROTOTYPES), OLX_PROTOTYPES)
    return _declare(lib, LOADER_EXTRA_PROTOTYPES)


def specialise_compile(program, row_program=False, dtype=HC_F32, cc=(10, 0)):
    """hcSpecialiseCompile: the device image NVRTC makes of ``program`` (an
    :class:`HcMapProgram`) for compute capability ``cc`` - no GPU needed.  Returns
    ``(image bytes, tag)``; raises RuntimeError with the library's message."""
    lib = load_kernels()
    message = C.create_string_buffer(8192)
    size = lib.hcSpecialiseCompile(C.byref(program), int(row_program), dtype, cc[0], cc[1], None,
                                   0, message, len(message))
    if size < 0:
        raise RuntimeError(message.value.decode(errors="replace"))
    image = C.create_string_buffer(size)
    size = lib.hcSpecialiseCompile(C.byref(program), int(row_program), dtype, cc[0], cc[1], image,
                                   size, message, len(message))
    if size < 0:
        raise RuntimeError(message.value.decode(errors="replace"))
    return image.raw[:size], message.value.decode()


def specialise_compile_items(code, dtype=HC_F32, group_threads=256, cc=(10, 0)):
    """hcSpecialiseCompileItems: the device image of a work-item program given by its
    instruction words, for work-groups of ``group_threads`` work-items - no GPU
    needed.  Returns ``(image bytes, tag)``."""
    lib = load_kernels()
    words = (C.c_uint32 * len(code))(*code)
    message = C.create_string_buffer(8192)
    size = lib.hcSpecialiseCompileItems(words, len(code), dtype, group_threads, cc[0], cc[1],
                                        None, 0, message, len(message))
    if size < 0:
        raise RuntimeError(message.value.decode(errors="replace"))
    image = C.create_string_buffer(size)
    size = lib.hcSpecialiseCompileItems(words, len(code), dtype, group_threads, cc[0], cc[1],
                                        image, size, message, len(message))
    if size < 0:
        raise RuntimeError(message.value.decode(errors="replace"))
    return image.raw[:size], message.value.decode()


def load_kernels():
    """libhc-b200-kernels.so (images + workload launchers)."""
    return _declare(_open("libhc-b200-kernels.so"), KERNELS_PROTOTYPES)


def load_python_runtime():
    """libhc-python-runtime.so (hcgpu*); holds the GIL while called."""
    return _declare(_open("libhc-python-runtime.so", C.PyDLL), PYRUNTIME_PROTOTYPES)


class HcError(RuntimeError):
    """A C-ABI call reported failure; the message is the library's own text."""


class Context:
    """Owns one HcContext and turns nonzero returns into :class:`HcError`.

    Arguments of the workload methods are raw device addresses (ints) and
    sizes, as in ``include/hc_b200_kernels.h``.
    """

    def __init__(self, device_desc: str = "cuda:0"):
        self.lib = load_kernels()
        self.messages = []

        def _on_message(_ctx, severity, text):
            self.messages.append((severity, (text or b"").decode(errors="replace")))

        self._callback = OlErrorCallback(_on_message)  # keep alive
        self.handle = self.lib.hcCreateContext(device_desc.encode(), self._callback, None)
        if not self.handle:
            errors = [m for s, m in self.messages if s == 0] or [m for _, m in self.messages]
            raise HcError(
                f"hcCreateContext({device_desc!r}) failed: " + ("; ".join(errors) or "no detail")
            )
        self.device_desc = device_desc

    def close(self):
        if getattr(self, "handle", None):
            self.lib.hcReleaseContext(self.handle)
            self.handle = None

    def __del__(self):  # pragma: no cover - best effort
        try:
            self.close()
        except Exception:
            pass

    def _check(self, rc, what):
        if rc:
            raise HcError(f"{what} failed: {self.lib.hcLastError(self.handle).decode(errors='replace')}")

    @property
    def stream(self) -> int:
        return self.lib.hcContextStream(self.handle) or 0

    @property
    def queue(self) -> int:
        return self.lib.hcContextQueue(self.handle)

    @property
    def device(self) -> int:
        return self.lib.hcContextDevice(self.handle)

    @property
    def launch_count(self) -> int:
        return self.lib.hcLaunchCount(self.handle)

    def synchronize(self):
        self._check(self.lib.hcSynchronize(self.handle), "hcSynchronize")

    def kernel_status(self) -> int:
        value = C.c_int(0)
        self._check(self.lib.hcKernelStatus(self.handle, C.byref(value)), "hcKernelStatus")
        return value.value

    def set_option(self, name: str, value: int):
        self._check(self.lib.hcSetOption(self.handle, name.encode(), value), "hcSetOption")

    def specialised_programs(self, from_disk: bool = False) -> int:
        """Programs this context compiled at run time (or loaded from the directory of
        HC_B200_KERNEL_CACHE)."""
        return self.lib.hcSpecialisedPrograms(self.handle, int(from_disk))

    @property
    def specialise_note(self) -> str:
        return (self.lib.hcSpecialiseNote(self.handle) or b"").decode()

    def copy2d(self, src, dst, rows, cols, src_pitch, dst_pitch, elem_bytes):
        self._check(
            self.lib.hcCopy2D(self.handle, src, dst, rows, cols, src_pitch, dst_pitch, elem_bytes),
            "hcCopy2D",
        )

    def softmax_rows(self, x, y, rows, cols, x_pitch, y_pitch, dtype=HC_F32):
        self._check(
            self.lib.hcSoftmaxRows(self.handle, x, y, rows, cols, x_pitch, y_pitch, dtype),
            "hcSoftmaxRows",
        )

    def reduce_rows(self, x, sum_out, max_out, rows, cols, pitch, dtype=HC_F32):
        self._check(
            self.lib.hcReduceRows(self.handle, x, sum_out, max_out, rows, cols, pitch, dtype),
            "hcReduceRows",
        )

    @staticmethod
    def _peers(bases):
        dsts = HcPeerOutputs()
        for d, base in enumerate(bases):
            dsts.base[d] = base
        dsts.count = len(bases)
        return dsts

    def softmax_rows_peers(self, x, bases, rows, cols, x_pitch, y_pitch, dtype=HC_F32):
        """``bases``: where this call's row 0 goes in every destination buffer."""
        self._check(
            self.lib.hcSoftmaxRowsPeers(self.handle, x, C.byref(self._peers(bases)), rows, cols,
                                        x_pitch, y_pitch, dtype),
            "hcSoftmaxRowsPeers",
        )

    def gemm_bf16_peers(self, a, b, bases, m, n, k, lda, ldb, ldc):
        self._check(
            self.lib.hcGemmBf16Peers(self.handle, a, b, C.byref(self._peers(bases)), m, n, k, lda,
                                     ldb, ldc),
            "hcGemmBf16Peers",
        )

    def gemm_w8a16_peers(self, a, w, scale, bases, workspace, workspace_bytes, m, n, k, lda, ldw,
                         ldc):
        self._check(
            self.lib.hcGemmW8A16Peers(self.handle, a, w, scale, C.byref(self._peers(bases)),
                                      workspace, workspace_bytes, m, n, k, lda, ldw, ldc),
            "hcGemmW8A16Peers",
        )

    def reduce_rows_peers(self, x, bases, max_offset, rows, cols, pitch, dtype=HC_F32):
        self._check(
            self.lib.hcReduceRowsPeers(self.handle, x, C.byref(self._peers(bases)), max_offset,
                                       rows, cols, pitch, dtype),
            "hcReduceRowsPeers",
        )

    def reduce_all(self, a, n, result, in_dtype=HC_F32, result_dtype=HC_F32):
        self._check(
            self.lib.hcReduceAll(self.handle, a, n, result, in_dtype, result_dtype), "hcReduceAll"
        )

    def pairwise_distance(self, a, b, out, m, n, d, lda, ldb, ldo, dtype=HC_F32):
        self._check(
            self.lib.hcPairwiseDistance(self.handle, a, b, out, m, n, d, lda, ldb, ldo, dtype),
            "hcPairwiseDistance",
        )

    def map_elements(self, program, dtype=HC_F32):
        """``program``: :class:`HcMapProgram`."""
        self._check(self.lib.hcMapElements(self.handle, C.byref(program), dtype), "hcMapElements")

    def work_items(self, program, dtype=HC_F32):
        """``program``: :class:`HcItemProgram`."""
        self._check(self.lib.hcWorkItems(self.handle, C.byref(program), dtype), "hcWorkItems")

    def row_program(self, program, dtype=HC_F32):
        """``program``: :class:`HcMapProgram` with row reductions."""
        self._check(self.lib.hcRowProgram(self.handle, C.byref(program), dtype), "hcRowProgram")

    def mapped_gemm(self, x, f, out, groups, tm, tn, k, dtype=HC_F32):
        """``x``, ``f``, ``out``: :class:`HcMappedOperand`."""
        self._check(
            self.lib.hcMappedGemm(self.handle, C.byref(x), C.byref(f), C.byref(out), groups,
                                  tm, tn, k, dtype),
            "hcMappedGemm",
        )

    def gemm_tiled(self, a, b, c, m, n, k, lda, ldb, ldc, dtype=HC_F32):
        self._check(
            self.lib.hcGemmTiled(self.handle, a, b, c, m, n, k, lda, ldb, ldc, dtype),
            "hcGemmTiled",
        )

    def conv_f32_tensor(self, x, f, out, n, c, h, w, nf, hf, wf, stride, workspace,
                        workspace_bytes):
        self._check(
            self.lib.hcConvF32Tensor(self.handle, x, f, out, n, c, h, w, nf, hf, wf, stride,
                                     workspace, workspace_bytes),
            "hcConvF32Tensor",
        )

    def gemm_f32_tensor(self, a, b, c, workspace, workspace_bytes, m, n, k, lda, ldb, ldc):
        self._check(
            self.lib.hcGemmF32Tensor(self.handle, a, b, c, workspace, workspace_bytes, m, n, k,
                                     lda, ldb, ldc),
            "hcGemmF32Tensor",
        )

    def gemm_bf16(self, a, b, c, m, n, k, lda, ldb, ldc):
        self._check(
            self.lib.hcGemmBf16(self.handle, a, b, c, m, n, k, lda, ldb, ldc), "hcGemmBf16"
        )

    def gemm_w8a16_workspace_bytes(self, n, k) -> int:
        return self.lib.hcGemmW8A16WorkspaceBytes(n, k)

    def gemm_w8a16_banded_bytes(self, n, k) -> int:
        return self.lib.hcGemmW8A16BandedBytes(n, k)

    def gemm_w8a16(self, a, w, scale, out, workspace, workspace_bytes, m, n, k, lda, ldw, ldc):
        self._check(
            self.lib.hcGemmW8A16(
                self.handle, a, w, scale, out, workspace, workspace_bytes, m, n, k, lda, ldw, ldc
            ),
            "hcGemmW8A16",
        )

    def gemm_w8a16_static(self, a, w, scale, out, m, n, k, lda, ldw, ldc):
        self._check(
            self.lib.hcGemmW8A16Static(self.handle, a, w, scale, out, m, n, k, lda, ldw, ldc),
            "hcGemmW8A16Static",
        )

    def host_pin(self, ptr, nbytes):
        self._check(self.lib.hcHostPin(self.handle, ptr, nbytes), "hcHostPin")

    def host_unpin(self, ptr):
        self._check(self.lib.hcHostUnpin(self.handle, ptr), "hcHostUnpin")

    def softmax_rows_host(self, x, y, rows, cols, x_pitch, y_pitch, dtype=HC_F32):
        """``x``, ``y``: HOST addresses."""
        self._check(
            self.lib.hcSoftmaxRowsHost(self.handle, x, y, rows, cols, x_pitch, y_pitch, dtype),
            "hcSoftmaxRowsHost",
        )

    def reduce_rows_host(self, x, sum_out, max_out, rows, cols, pitch, dtype=HC_F32):
        self._check(
            self.lib.hcReduceRowsHost(self.handle, x, sum_out, max_out, rows, cols, pitch, dtype),
            "hcReduceRowsHost",
        )

    def gemm_bf16_host(self, a, b, c, m, n, k, lda, ldb, ldc):
        self._check(
            self.lib.hcGemmBf16Host(self.handle, a, b, c, m, n, k, lda, ldb, ldc),
            "hcGemmBf16Host",
        )

    def dequant_w8(self, w, out, rows, cols, w_pitch, out_pitch):
        self._check(
            self.lib.hcDequantW8(self.handle, w, out, rows, cols, w_pitch, out_pitch),
            "hcDequantW8",
        )
