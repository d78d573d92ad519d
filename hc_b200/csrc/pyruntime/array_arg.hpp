// Reads pointer, shape, strides and element type out of an array-like Python
// object without depending on any array library at build time.
//
// Accepted, in this order:
//   * objects with data_ptr()/shape/stride()/element_size()/dtype - torch
//     tensors (the reference's e2e tests pass torch CUDA tensors,
//     python/hckernel/tests/test_e2e.py:72-75).  torch refuses to export bf16
//     through __cuda_array_interface__, so this branch comes first;
//   * objects with __cuda_array_interface__ (CuPy, Numba device arrays);
//   * objects with __array_interface__ (NumPy) - host memory.
// The reference does the same job with nanobind's ndarray caster
// (python/cpp/py-runtime/src/PyABI.cpp:23-37).
#pragma once

#include <pybind11/pybind11.h>

#include <cstdint>
#include <stdexcept>
#include <string>
#include <vector>

namespace hc {

namespace py = pybind11;

enum class ElemKind { F32, F64, BF16, F16, I8, U8, I16, I32, I64, Other };

struct ArrayArg {
  void *data = nullptr;
  std::vector<int64_t> shape;
  std::vector<int64_t> strides; // in elements
  int64_t itemsize = 0;
  ElemKind kind = ElemKind::Other;
  bool onDevice = false;
  int deviceIndex = -1; // -1: unknown or host

  int rank() const { return int(shape.size()); }
  // Rows are contiguous (last stride 1) - what every kernel here requires.
  bool rowMajor() const { return shape.empty() || strides.back() == 1 || shape.back() <= 1; }
};

inline const char *kindName(ElemKind k) {
  switch (k) {
  case ElemKind::F32: return "float32";
  case ElemKind::F64: return "float64";
  case ElemKind::BF16: return "bfloat16";
  case ElemKind::F16: return "float16";
  case ElemKind::I8: return "int8";
  case ElemKind::U8: return "uint8";
  case ElemKind::I16: return "int16";
  case ElemKind::I32: return "int32";
  case ElemKind::I64: return "int64";
  default: return "other";
  }
}

inline ElemKind kindFromTorchName(const std::string &name) {
  // str(tensor.dtype) is "torch.float32" etc.
  auto dot = name.rfind('.');
  std::string n = dot == std::string::npos ? name : name.substr(dot + 1);
  if (n == "float32" || n == "float") return ElemKind::F32;
  if (n == "float64" || n == "double") return ElemKind::F64;
  if (n == "bfloat16") return ElemKind::BF16;
  if (n == "float16" || n == "half") return ElemKind::F16;
  if (n == "int8") return ElemKind::I8;
  if (n == "uint8") return ElemKind::U8;
  if (n == "int16" || n == "short") return ElemKind::I16;
  if (n == "int32" || n == "int") return ElemKind::I32;
  if (n == "int64" || n == "long") return ElemKind::I64;
  return ElemKind::Other;
}

inline ElemKind kindFromTypestr(const std::string &t, int64_t &itemsize) {
  // "<f4", "|i1", "<u2", ...
  if (t.size() < 3)
    return ElemKind::Other;
  char c = t[1];
  itemsize = std::stoll(t.substr(2));
  if (c == 'f') return itemsize == 4 ? ElemKind::F32 : itemsize == 8 ? ElemKind::F64
                     : itemsize == 2 ? ElemKind::F16 : ElemKind::Other;
  if (c == 'i') return itemsize == 1 ? ElemKind::I8 : itemsize == 2 ? ElemKind::I16
                     : itemsize == 4 ? ElemKind::I32 : itemsize == 8 ? ElemKind::I64
                     : ElemKind::Other;
  if (c == 'u') return itemsize == 1 ? ElemKind::U8 : ElemKind::Other;
  return ElemKind::Other;
}

inline ArrayArg arrayFromInterface(const py::dict &iface, bool onDevice) {
  ArrayArg a;
  a.onDevice = onDevice;
  auto data = iface["data"].cast<py::tuple>();
  a.data = reinterpret_cast<void *>(data[0].cast<uintptr_t>());
  a.kind = kindFromTypestr(iface["typestr"].cast<std::string>(), a.itemsize);
  for (auto d : iface["shape"].cast<py::tuple>())
    a.shape.push_back(d.cast<int64_t>());
  bool haveStrides = iface.contains("strides") && !iface["strides"].is_none();
  if (haveStrides) {
    for (auto s : iface["strides"].cast<py::tuple>()) {
      int64_t bytes = s.cast<int64_t>();
      if (a.itemsize == 0 || bytes % a.itemsize)
        throw std::runtime_error("Array strides are not a multiple of the element size");
      a.strides.push_back(bytes / a.itemsize);
    }
  } else {
    a.strides.assign(a.shape.size(), 1);
    for (int i = int(a.shape.size()) - 2; i >= 0; --i)
      a.strides[i] = a.strides[i + 1] * a.shape[i + 1];
  }
  return a;
}

inline ArrayArg arrayFromPython(py::handle obj) {
  if (py::hasattr(obj, "data_ptr") && py::hasattr(obj, "element_size")) {
    ArrayArg a;
    a.data = reinterpret_cast<void *>(obj.attr("data_ptr")().cast<uintptr_t>());
    for (auto d : obj.attr("shape"))
      a.shape.push_back(d.cast<int64_t>());
    for (auto s : obj.attr("stride")())
      a.strides.push_back(s.cast<int64_t>());
    a.itemsize = obj.attr("element_size")().cast<int64_t>();
    a.kind = kindFromTorchName(py::str(obj.attr("dtype")).cast<std::string>());
    a.onDevice = obj.attr("is_cuda").cast<bool>();
    if (a.onDevice) {
      py::object idx = obj.attr("device").attr("index");
      a.deviceIndex = idx.is_none() ? 0 : idx.cast<int>();
    }
    return a;
  }
  if (py::hasattr(obj, "__cuda_array_interface__"))
    return arrayFromInterface(obj.attr("__cuda_array_interface__").cast<py::dict>(), true);
  if (py::hasattr(obj, "__array_interface__"))
    return arrayFromInterface(obj.attr("__array_interface__").cast<py::dict>(), false);
  throw std::runtime_error("Object is not an array (no data_ptr, __cuda_array_interface__ "
                           "or __array_interface__)");
}

} // namespace hc
