// hc_b200._native._dispatcher: the Python entry of the launch path.
//
// In the reference a call of a @kernel-decorated function lands in a nanobind
// Dispatcher that checks the arguments, builds a specialization key, JIT
// compiles on a miss and calls the compiled host wrapper
// (python/cpp/compiler/src/DispatcherBase.cpp:250-280, 542-585;
// python/cpp/compiler/src/Dispatcher.cpp:20-42).  The JIT is gone here, so what
// remains is argument checking and the call into the precompiled kernels:
// every function below reads its array arguments (array_arg.hpp), validates
// device, element type, rank and layout, and forwards to one entry point of
// libhc-b200-kernels.so.  Validation errors raise ValueError/TypeError, launch
// errors RuntimeError with the library's own message - never abort().
#include "array_arg.hpp"
#include "hc_b200_kernels.h"

#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <algorithm>
#include <array>
#include <charconv>
#include <memory>
#include <string>
#include <vector>

namespace py = pybind11;
using hc::ArrayArg;
using hc::ElemKind;

namespace {

class Context {
public:
  explicit Context(const std::string &desc) : description(desc) {
    handle = hcCreateContext(desc.c_str(), &Context::onMessage, this);
    if (!handle)
      throw std::runtime_error("cannot open device '" + desc + "': " +
                               (errors.empty() ? "no detail" : errors));
    auto colon = desc.find(':');
    if (colon != std::string::npos)
      std::from_chars(desc.data() + colon + 1, desc.data() + desc.size(), ordinal);
  }
  ~Context() { close(); }
  Context(const Context &) = delete;
  Context &operator=(const Context &) = delete;

  void close() {
    if (handle)
      hcReleaseContext(handle);
    handle = nullptr;
  }

  HcContext get() const {
    if (!handle)
      throw std::runtime_error("context is closed");
    return handle;
  }

  void check(int rc, const char *what) const {
    if (rc)
      throw std::runtime_error(std::string(what) + " failed: " + hcLastError(handle));
  }

  std::string description;
  int ordinal = 0;

private:
  static void onMessage(void *self, OlSeverity sev, const char *text) {
    auto *c = static_cast<Context *>(self);
    if (sev == OlSeverity::Error) {
      if (!c->errors.empty())
        c->errors += "; ";
      c->errors += text ? text : "";
    }
  }
  HcContext handle = nullptr;
  std::string errors;
};

// Reads an argument and checks what every kernel needs: device memory on the
// context's GPU, the expected rank, contiguous rows.
ArrayArg deviceArray(const Context &ctx, py::handle obj, const char *name,
                     int rank) {
  ArrayArg a;
  try {
    a = hc::arrayFromPython(obj);
  } catch (const std::exception &e) {
    throw py::type_error(std::string(name) + ": " + e.what());
  }
  if (!a.onDevice)
    throw py::value_error(std::string(name) +
                          ": expected device memory (a CUDA tensor), got host memory");
  if (a.deviceIndex >= 0 && a.deviceIndex != ctx.ordinal)
    throw py::value_error(std::string(name) + ": lives on cuda:" +
                          std::to_string(a.deviceIndex) + " but the kernel runs on " +
                          ctx.description);
  if (a.rank() != rank)
    throw py::value_error(std::string(name) + ": expected rank " + std::to_string(rank) +
                          ", got " + std::to_string(a.rank()));
  if (!a.rowMajor())
    throw py::value_error(std::string(name) + ": rows must be contiguous (last stride 1)");
  for (auto s : a.strides)
    if (s < 0)
      throw py::value_error(std::string(name) + ": negative strides are not supported");
  return a;
}

void sameKind(const ArrayArg &a, const ArrayArg &b, const char *an, const char *bn) {
  if (a.kind != b.kind || a.itemsize != b.itemsize)
    throw py::type_error(std::string(an) + " is " + hc::kindName(a.kind) + " but " + bn +
                         " is " + hc::kindName(b.kind));
}

void sameShape(const ArrayArg &a, const ArrayArg &b, const char *an, const char *bn) {
  if (a.shape != b.shape)
    throw py::value_error(std::string(an) + " and " + bn + " differ in shape");
}

long long pitch(const ArrayArg &a) {
  // Row pitch of a rank-2 array; a single row may report any stride.
  return a.shape[0] > 1 ? a.strides[0] : std::max<long long>(a.strides[0], a.shape[1]);
}

int floatDType(const ArrayArg &a, const char *name) {
  if (a.kind == ElemKind::F32)
    return HC_F32;
  if (a.kind == ElemKind::F64)
    return HC_F64;
  throw py::type_error(std::string(name) + ": float32 or float64 expected, got " +
                       hc::kindName(a.kind));
}

void copy2d(Context &ctx, py::handle src, py::handle dst) {
  ArrayArg s = deviceArray(ctx, src, "src", 2), d = deviceArray(ctx, dst, "dst", 2);
  sameKind(s, d, "src", "dst");
  sameShape(s, d, "src", "dst");
  ctx.check(hcCopy2D(ctx.get(), s.data, d.data, s.shape[0], s.shape[1], pitch(s), pitch(d),
                     int(s.itemsize)),
            "copy2d");
}

void softmaxRows(Context &ctx, py::handle x, py::handle y) {
  ArrayArg a = deviceArray(ctx, x, "x", 2), b = deviceArray(ctx, y, "out", 2);
  sameKind(a, b, "x", "out");
  sameShape(a, b, "x", "out");
  ctx.check(hcSoftmaxRows(ctx.get(), a.data, b.data, a.shape[0], a.shape[1], pitch(a),
                          pitch(b), floatDType(a, "x")),
            "softmax_rows");
}

void reduceRows(Context &ctx, py::handle x, py::object sumOut, py::object maxOut) {
  ArrayArg a = deviceArray(ctx, x, "x", 2);
  int dtype = floatDType(a, "x");
  void *sp = nullptr, *mp = nullptr;
  auto output = [&](py::object &o, const char *name) -> void * {
    if (o.is_none())
      return nullptr;
    ArrayArg r = deviceArray(ctx, o, name, 1);
    sameKind(a, r, "x", name);
    if (r.shape[0] != a.shape[0])
      throw py::value_error(std::string(name) + ": expected " +
                            std::to_string(a.shape[0]) + " elements");
    if (r.shape[0] > 1 && r.strides[0] != 1)
      throw py::value_error(std::string(name) + ": must be contiguous");
    return r.data;
  };
  sp = output(sumOut, "sum_out");
  mp = output(maxOut, "max_out");
  ctx.check(hcReduceRows(ctx.get(), a.data, sp, mp, a.shape[0], a.shape[1], pitch(a), dtype),
            "reduce_rows");
}

// ---- host buffers (hcSoftmaxRowsHost, hcReduceRowsHost, hcGemmBf16Host) ---------------
// A host array (a NumPy array or a CPU tensor; page-locked memory makes the
// copies overlap), rows contiguous.
ArrayArg hostArray(py::handle obj, const char *name, int rank) {
  ArrayArg a;
  try {
    a = hc::arrayFromPython(obj);
  } catch (const std::exception &e) {
    throw py::type_error(std::string(name) + ": " + e.what());
  }
  if (a.onDevice)
    throw py::value_error(std::string(name) + ": expected host memory, got a CUDA tensor");
  if (a.rank() != rank)
    throw py::value_error(std::string(name) + ": expected rank " + std::to_string(rank) +
                          ", got " + std::to_string(a.rank()));
  if (!a.rowMajor())
    throw py::value_error(std::string(name) + ": rows must be contiguous (last stride 1)");
  for (auto s : a.strides)
    if (s < 0)
      throw py::value_error(std::string(name) + ": negative strides are not supported");
  return a;
}

void softmaxRowsHost(Context &ctx, py::handle x, py::handle y) {
  ArrayArg a = hostArray(x, "x", 2), b = hostArray(y, "out", 2);
  sameKind(a, b, "x", "out");
  sameShape(a, b, "x", "out");
  const int dtype = floatDType(a, "x");
  int rc;
  {
    py::gil_scoped_release release; // the call waits for the GPU
    rc = hcSoftmaxRowsHost(ctx.get(), a.data, b.data, a.shape[0], a.shape[1], pitch(a), pitch(b),
                           dtype);
  }
  ctx.check(rc, "softmax_rows_host");
}

void reduceRowsHost(Context &ctx, py::handle x, py::object sumOut, py::object maxOut) {
  ArrayArg a = hostArray(x, "x", 2);
  const int dtype = floatDType(a, "x");
  auto output = [&](py::object &o, const char *name) -> void * {
    if (o.is_none())
      return nullptr;
    ArrayArg r = hostArray(o, name, 1);
    sameKind(a, r, "x", name);
    if (r.shape[0] != a.shape[0] || (r.shape[0] > 1 && r.strides[0] != 1))
      throw py::value_error(std::string(name) + ": expected " + std::to_string(a.shape[0]) +
                            " contiguous elements");
    return r.data;
  };
  void *sp = output(sumOut, "sum_out"), *mp = output(maxOut, "max_out");
  int rc;
  {
    py::gil_scoped_release release;
    rc = hcReduceRowsHost(ctx.get(), a.data, sp, mp, a.shape[0], a.shape[1], pitch(a), dtype);
  }
  ctx.check(rc, "reduce_rows_host");
}

void gemmBf16Host(Context &ctx, py::handle a, py::handle b, py::handle out) {
  ArrayArg A = hostArray(a, "a", 2), B = hostArray(b, "b", 2), O = hostArray(out, "out", 2);
  if (A.kind != ElemKind::BF16 || B.kind != ElemKind::BF16 || O.kind != ElemKind::BF16)
    throw py::type_error("gemm_bf16_host: bfloat16 matrices expected");
  if (A.shape[1] != B.shape[0] || O.shape[0] != A.shape[0] || O.shape[1] != B.shape[1])
    throw py::value_error("gemm_bf16_host: shapes do not form [M,K] @ [K,N] -> [M,N]");
  int rc;
  {
    py::gil_scoped_release release;
    rc = hcGemmBf16Host(ctx.get(), A.data, B.data, O.data, A.shape[0], B.shape[1], A.shape[1],
                        pitch(A), pitch(B), pitch(O));
  }
  ctx.check(rc, "gemm_bf16_host");
}

// The same two workloads writing their rows into every rank's output buffer
// (hcSoftmaxRowsPeers, hcReduceRowsPeers): `bases` are raw device addresses -
// this GPU's memory or peer memory mapped into the process - of where the
// call's row 0 goes in each destination.
HcPeerOutputs peerOutputs(const std::vector<uintptr_t> &bases) {
  if (bases.empty() || bases.size() > 8)
    throw py::value_error("1..8 destination addresses expected");
  HcPeerOutputs dsts{};
  for (size_t d = 0; d < bases.size(); ++d)
    dsts.base[d] = reinterpret_cast<void *>(bases[d]);
  dsts.count = int(bases.size());
  return dsts;
}

void softmaxRowsPeers(Context &ctx, py::handle x, const std::vector<uintptr_t> &bases,
                      long long outPitch) {
  ArrayArg a = deviceArray(ctx, x, "x", 2);
  HcPeerOutputs dsts = peerOutputs(bases);
  ctx.check(hcSoftmaxRowsPeers(ctx.get(), a.data, &dsts, a.shape[0], a.shape[1], pitch(a),
                               outPitch, floatDType(a, "x")),
            "softmax_rows_peers");
}

void gemmBf16Peers(Context &ctx, py::handle a, py::handle b, const std::vector<uintptr_t> &bases,
                   long long outPitch) {
  ArrayArg A = deviceArray(ctx, a, "a", 2), B = deviceArray(ctx, b, "b", 2);
  if (A.kind != ElemKind::BF16 || B.kind != ElemKind::BF16)
    throw py::type_error("gemm_bf16_peers: bfloat16 matrices expected");
  if (A.shape[1] != B.shape[0])
    throw py::value_error("gemm_bf16_peers: shapes do not form [M,K] @ [K,N]");
  HcPeerOutputs dsts = peerOutputs(bases);
  ctx.check(hcGemmBf16Peers(ctx.get(), A.data, B.data, &dsts, A.shape[0], B.shape[1], A.shape[1],
                            pitch(A), pitch(B), outPitch),
            "gemm_bf16_peers");
}

void gemmW8A16Peers(Context &ctx, py::handle a, py::handle w, py::handle scale,
                    const std::vector<uintptr_t> &bases, long long outPitch,
                    py::handle workspace) {
  ArrayArg A = deviceArray(ctx, a, "a", 2), W = deviceArray(ctx, w, "w", 2),
           S = deviceArray(ctx, scale, "scale", 1), ws = deviceArray(ctx, workspace, "workspace", 1);
  if (A.kind != ElemKind::BF16 || W.kind != ElemKind::I8 || S.kind != ElemKind::F32)
    throw py::type_error("gemm_w8a16_peers: a bfloat16, w int8, scale float32 expected");
  if (A.shape[1] != W.shape[0] || S.shape[0] != W.shape[1])
    throw py::value_error("gemm_w8a16_peers: shapes do not form [M,K] @ [K,N] with scale [N]");
  HcPeerOutputs dsts = peerOutputs(bases);
  ctx.check(hcGemmW8A16Peers(ctx.get(), A.data, W.data, static_cast<const float *>(S.data), &dsts,
                             ws.data, size_t(ws.shape[0]) * size_t(ws.itemsize), A.shape[0],
                             W.shape[1], A.shape[1], pitch(A), pitch(W), outPitch),
            "gemm_w8a16_peers");
}

void reduceRowsPeers(Context &ctx, py::handle x, const std::vector<uintptr_t> &bases,
                     long long maxOffset) {
  ArrayArg a = deviceArray(ctx, x, "x", 2);
  HcPeerOutputs dsts = peerOutputs(bases);
  ctx.check(hcReduceRowsPeers(ctx.get(), a.data, &dsts, maxOffset, a.shape[0], a.shape[1],
                              pitch(a), floatDType(a, "x")),
            "reduce_rows_peers");
}

void reduceAll(Context &ctx, py::handle a, py::handle result) {
  ArrayArg A = deviceArray(ctx, a, "a", 1), R = deviceArray(ctx, result, "result", 1);
  if (A.shape[0] > 1 && A.strides[0] != 1)
    throw py::value_error("a: must be contiguous");
  if (R.shape[0] < 1)
    throw py::value_error("result: needs at least one element");
  int in = A.kind == ElemKind::F32   ? HC_F32
           : A.kind == ElemKind::F64 ? HC_F64
           : A.kind == ElemKind::I32 ? HC_I32
           : A.kind == ElemKind::I64 ? HC_I64
                                     : -1;
  if (in < 0)
    throw py::type_error(std::string("a: float32, float64, int32 or int64 expected, got ") +
                         hc::kindName(A.kind));
  ctx.check(hcReduceAll(ctx.get(), A.data, A.shape[0], R.data, in, floatDType(R, "result")),
            "reduce_all");
}

void pairwiseDistance(Context &ctx, py::handle a, py::handle b, py::handle out) {
  ArrayArg A = deviceArray(ctx, a, "a", 2), B = deviceArray(ctx, b, "b", 2),
           O = deviceArray(ctx, out, "out", 2);
  sameKind(A, B, "a", "b");
  sameKind(A, O, "a", "out");
  if (A.shape[1] != B.shape[1] || O.shape[0] != A.shape[0] || O.shape[1] != B.shape[0])
    throw py::value_error("pairwise_distance: shapes do not form [M,D], [N,D] -> [M,N]");
  ctx.check(hcPairwiseDistance(ctx.get(), A.data, B.data, O.data, A.shape[0], B.shape[0],
                               A.shape[1], pitch(A), pitch(B), pitch(O), floatDType(A, "a")),
            "pairwise_distance");
}

// Element-wise expression over matrices (or vectors) of one shape and type:
// `inputs` a list of up to four arrays, `code` and `consts` the program
// (include/hc_b200_kernels.h: HcMapProgram).
void runProgram(Context &ctx, py::handle inputs, py::handle out, const std::vector<unsigned> &code,
                const std::vector<double> &consts, bool rowProgram) {
  auto ins = py::cast<py::list>(inputs);
  if (ins.size() > 4)
    throw py::value_error("map_elements: at most 4 input arrays");
  if (code.empty() || code.size() > 32 || consts.size() > 8)
    throw py::value_error("map_elements: 1..32 instructions and at most 8 constants");
  ArrayArg o;
  try {
    o = hc::arrayFromPython(out);
  } catch (const std::exception &e) {
    throw py::type_error(std::string("out: ") + e.what());
  }
  const int rank = o.rank();
  if (rank != 1 && rank != 2)
    throw py::value_error("map_elements: vectors or matrices expected");
  ArrayArg O = deviceArray(ctx, out, "out", rank);
  HcMapProgram p{};
  auto rows = [&](const ArrayArg &a) { return rank == 2 ? a.shape[0] : 1; };
  auto cols = [&](const ArrayArg &a) { return a.shape[rank - 1]; };
  auto rowPitch = [&](const ArrayArg &a) { return rank == 2 ? pitch(a) : a.shape[0]; };
  p.out = O.data;
  p.outPitch = rowPitch(O);
  p.rows = rows(O);
  p.cols = cols(O);
  p.nInputs = int(ins.size());
  for (int k = 0; k < p.nInputs; ++k) {
    const std::string name = "input " + std::to_string(k);
    ArrayArg a = deviceArray(ctx, ins[k], name.c_str(), rank);
    sameKind(a, O, name.c_str(), "out");
    sameShape(a, O, name.c_str(), "out");
    p.in[k] = a.data;
    p.inPitch[k] = rowPitch(a);
  }
  p.nInstr = int(code.size());
  std::copy(code.begin(), code.end(), p.code);
  std::copy(consts.begin(), consts.end(), p.consts);
  if (rowProgram) {
    if (rank != 2)
      throw py::value_error("row_program: matrices expected");
    ctx.check(hcRowProgram(ctx.get(), &p, floatDType(O, "out")), "row_program");
  } else {
    const int dtype = O.kind == ElemKind::I32   ? HC_I32
                      : O.kind == ElemKind::I64 ? HC_I64
                                                : floatDType(O, "out");
    ctx.check(hcMapElements(ctx.get(), &p, dtype), "map_elements");
  }
}

void mapElements(Context &ctx, py::handle inputs, py::handle out, const std::vector<unsigned> &code,
                 const std::vector<double> &consts) {
  runProgram(ctx, inputs, out, code, consts, false);
}

// Work-item program (hcWorkItems): `inputs` arrays of the shape of `out`, each
// read at the work-item's global id plus `offsets[k]` = (row, column); `group`
// the work-group shape (rows, columns); `guards` one (lo row, hi row, lo column,
// hi column) per phase; `tiles` the reads of the group's tile as (row scale, row
// offset, row wrap, column scale, column offset, column wrap).
void workItems(Context &ctx, py::handle inputs, const std::vector<std::pair<int, int>> &offsets,
               py::handle out, std::pair<int, int> group, const std::vector<unsigned> &code,
               const std::vector<double> &consts,
               const std::vector<std::array<long long, 4>> &guards,
               const std::vector<std::array<int, 6>> &tiles, double tileFill) {
  auto ins = py::cast<py::list>(inputs);
  if (ins.size() > 4 || offsets.size() != ins.size())
    throw py::value_error("work_items: at most 4 input arrays, one offset pair each");
  if (code.empty() || code.size() > 48 || consts.size() > 8 || guards.empty() ||
      guards.size() > 2 || tiles.size() > 4)
    throw py::value_error("work_items: 1..48 instructions, at most 8 constants, 1..2 guards and "
                          "at most 4 tile reads");
  ArrayArg o;
  try {
    o = hc::arrayFromPython(out);
  } catch (const std::exception &e) {
    throw py::type_error(std::string("out: ") + e.what());
  }
  const int rank = o.rank();
  if (rank != 1 && rank != 2)
    throw py::value_error("work_items: vectors or matrices expected");
  ArrayArg O = deviceArray(ctx, out, "out", rank);
  HcItemProgram p{};
  auto rowPitch = [&](const ArrayArg &a) { return rank == 2 ? pitch(a) : a.shape[0]; };
  p.out = O.data;
  p.outPitch = rowPitch(O);
  p.rows = rank == 2 ? O.shape[0] : 1;
  p.cols = O.shape[rank - 1];
  p.groupRows = group.first;
  p.groupCols = group.second;
  p.nInputs = int(ins.size());
  for (int k = 0; k < p.nInputs; ++k) {
    const std::string name = "input " + std::to_string(k);
    ArrayArg a = deviceArray(ctx, ins[k], name.c_str(), rank);
    sameKind(a, O, name.c_str(), "out");
    sameShape(a, O, name.c_str(), "out");
    p.in[k] = a.data;
    p.inPitch[k] = rowPitch(a);
    p.inRow[k] = offsets[k].first;
    p.inCol[k] = offsets[k].second;
  }
  p.nInstr = int(code.size());
  std::copy(code.begin(), code.end(), p.code);
  std::copy(consts.begin(), consts.end(), p.consts);
  for (size_t ph = 0; ph < 2; ++ph) {
    const auto &g = guards[std::min(ph, guards.size() - 1)];
    p.guardLo[ph][0] = g[0];
    p.guardHi[ph][0] = g[1];
    p.guardLo[ph][1] = g[2];
    p.guardHi[ph][1] = g[3];
  }
  for (size_t k = 0; k < tiles.size(); ++k) {
    p.tileScale[k][0] = tiles[k][0];
    p.tileOffset[k][0] = tiles[k][1];
    p.tileMod[k][0] = tiles[k][2];
    p.tileScale[k][1] = tiles[k][3];
    p.tileOffset[k][1] = tiles[k][4];
    p.tileMod[k][1] = tiles[k][5];
  }
  p.tileFill = tileFill;
  ctx.check(hcWorkItems(ctx.get(), &p, floatDType(O, "out")), "work_items");
}

// Row program (hcRowProgram): like map_elements, with reductions along the rows.
void rowProgram(Context &ctx, py::handle inputs, py::handle out, const std::vector<unsigned> &code,
                const std::vector<double> &consts) {
  runProgram(ctx, inputs, out, code, consts, true);
}

// One operand of the gathered tile product: the array (any rank up to 4, any
// non-negative strides) and its tables (map int32 [E,4], lin int32 [E],
// origins int32 [G,4], lo and hi as 4 ints each, whether map/lin are in
// transposed tile order).
HcMappedOperand mappedOperand(const Context &ctx, py::handle array, py::handle tables,
                              const char *name, long long elems, long long groups,
                              ElemKind *kind) {
  ArrayArg a;
  try {
    a = hc::arrayFromPython(array);
  } catch (const std::exception &e) {
    throw py::type_error(std::string(name) + ": " + e.what());
  }
  if (!a.onDevice)
    throw py::value_error(std::string(name) + ": expected device memory (a CUDA tensor)");
  if (a.deviceIndex >= 0 && a.deviceIndex != ctx.ordinal)
    throw py::value_error(std::string(name) + ": lives on another GPU than " + ctx.description);
  if (a.rank() < 1 || a.rank() > 4)
    throw py::value_error(std::string(name) + ": rank 1 to 4 expected");
  *kind = a.kind;
  HcMappedOperand op{};
  op.base = a.data;
  for (int d = 0; d < 4; ++d) {
    op.shape[d] = 1;
    op.stride[d] = 0;
  }
  for (int d = 0; d < a.rank(); ++d) {
    if (a.strides[d] < 0 || a.shape[d] > 0x7fffffffLL)
      throw py::value_error(std::string(name) + ": negative stride or extent above 2^31");
    op.shape[d] = int(a.shape[d]);
    op.stride[d] = a.strides[d];
  }
  auto t = py::cast<py::tuple>(tables);
  if (t.size() != 7)
    throw py::value_error(std::string(name) +
                          ": tables must be (map, lin, origins, lo, hi, transposed, shared_run)");
  op.transposed = py::cast<bool>(t[5]) ? 1 : 0;
  op.sharedRun = py::cast<int>(t[6]);
  const std::string nm(name);
  ArrayArg map = deviceArray(ctx, t[0], (nm + " map").c_str(), 2);
  ArrayArg lin = deviceArray(ctx, t[1], (nm + " lin").c_str(), 1);
  ArrayArg org = deviceArray(ctx, t[2], (nm + " origins").c_str(), 2);
  for (const ArrayArg *tab : {&map, &lin, &org})
    if (tab->kind != ElemKind::I32)
      throw py::type_error(nm + ": tables must be int32");
  if (map.shape[0] != elems || map.shape[1] != 4 || (elems > 1 && map.strides[0] != 4) ||
      lin.shape[0] != elems)
    throw py::value_error(nm + ": map/lin tables do not match the tile");
  if (org.shape[0] != groups || org.shape[1] != 4 || (groups > 1 && org.strides[0] != 4))
    throw py::value_error(nm + ": origins table does not match the work-groups");
  op.map = static_cast<const int *>(map.data);
  op.lin = static_cast<const int *>(lin.data);
  op.origins = static_cast<const int *>(org.data);
  auto lo = py::cast<std::vector<int>>(t[3]), hi = py::cast<std::vector<int>>(t[4]);
  if (lo.size() != 4 || hi.size() != 4)
    throw py::value_error(nm + ": lo and hi must have 4 entries");
  for (int d = 0; d < 4; ++d) {
    op.lo[d] = lo[d];
    op.hi[d] = hi[d];
  }
  return op;
}

void mappedGemm(Context &ctx, py::handle x, py::handle xTables, py::handle f,
                py::handle fTables, py::handle out, py::handle outTables, long long groups,
                int tm, int tn, int k) {
  if (groups < 0 || tm < 0 || tn < 0 || k < 0)
    throw py::value_error("mapped_gemm: negative size");
  ElemKind kx, kf, ko;
  HcMappedOperand X = mappedOperand(ctx, x, xTables, "x", (long long)tm * k, groups, &kx);
  HcMappedOperand F = mappedOperand(ctx, f, fTables, "f", (long long)k * tn, groups, &kf);
  HcMappedOperand O = mappedOperand(ctx, out, outTables, "out", (long long)tm * tn, groups, &ko);
  if (kx != kf || kx != ko)
    throw py::type_error("mapped_gemm: x, f and out differ in element type");
  if (kx != ElemKind::F32 && kx != ElemKind::F64)
    throw py::type_error(std::string("mapped_gemm: float32 or float64 expected, got ") +
                         hc::kindName(kx));
  ctx.check(hcMappedGemm(ctx.get(), &X, &F, &O, groups, tm, tn, k,
                         kx == ElemKind::F32 ? HC_F32 : HC_F64),
            "mapped_gemm");
}

size_t gemmF32WorkspaceBytes(long long m, long long n, long long k) {
  return hcGemmF32TensorWorkspaceBytes(m, n, k);
}

// float32 convolution without padding on the tensor cores (hcConvF32Tensor):
// x [N, C, H, W], f [NF, C, HF, WF], out [N, NF, HO, WO], all contiguous.
size_t convF32WorkspaceBytes(long long n, long long c, long long h, long long w, long long nf,
                             long long hf, long long wf) {
  return hcConvF32TensorWorkspaceBytes(n, c, h, w, nf, hf, wf);
}

bool contiguous(const ArrayArg &a) {
  long long expect = 1;
  for (int d = a.rank() - 1; d >= 0; --d) {
    if (a.shape[d] > 1 && a.strides[d] != expect)
      return false;
    expect *= a.shape[d];
  }
  return true;
}

void convF32Tensor(Context &ctx, py::handle x, py::handle f, py::handle out, long long stride,
                   py::handle workspace) {
  ArrayArg X = deviceArray(ctx, x, "x", 4), F = deviceArray(ctx, f, "f", 4),
           O = deviceArray(ctx, out, "out", 4);
  ArrayArg ws = deviceArray(ctx, workspace, "workspace", 1);
  if (X.kind != ElemKind::F32 || F.kind != ElemKind::F32 || O.kind != ElemKind::F32)
    throw py::type_error("conv_f32_tensor: float32 arrays");
  if (!contiguous(X) || !contiguous(F) || !contiguous(O))
    throw py::value_error("conv_f32_tensor: x, f and out must be contiguous");
  if (stride < 1 || F.shape[1] != X.shape[1] || F.shape[2] > X.shape[2] ||
      F.shape[3] > X.shape[3])
    throw py::value_error("conv_f32_tensor: shapes do not form a convolution");
  const long long ho = (X.shape[2] - F.shape[2]) / stride + 1,
                  wo = (X.shape[3] - F.shape[3]) / stride + 1;
  if (O.shape[0] != X.shape[0] || O.shape[1] != F.shape[0] || O.shape[2] != ho ||
      O.shape[3] != wo)
    throw py::value_error("conv_f32_tensor: out must be [N, NF, (H-HF)/stride+1, "
                          "(W-WF)/stride+1]");
  ctx.check(hcConvF32Tensor(ctx.get(), X.data, F.data, O.data, X.shape[0], X.shape[1],
                            X.shape[2], X.shape[3], F.shape[0], F.shape[2], F.shape[3], stride,
                            ws.data, size_t(ws.shape[0]) * size_t(ws.itemsize)),
            "conv_f32_tensor");
}

// `workspace` (a uint8 device buffer of gemm_f32_workspace_bytes) sends a
// float32 product to the tensor cores (hcGemmF32Tensor).
void gemm(Context &ctx, py::handle a, py::handle b, py::handle out, py::object workspace) {
  ArrayArg A = deviceArray(ctx, a, "a", 2), B = deviceArray(ctx, b, "b", 2),
           C = deviceArray(ctx, out, "out", 2);
  sameKind(A, B, "a", "b");
  sameKind(A, C, "a", "out");
  long long M = A.shape[0], K = A.shape[1], N = B.shape[1];
  if (B.shape[0] != K || C.shape[0] != M || C.shape[1] != N)
    throw py::value_error("gemm: shapes do not form [M,K] @ [K,N] -> [M,N]");
  if (A.kind == ElemKind::BF16) {
    ctx.check(hcGemmBf16(ctx.get(), A.data, B.data, C.data, M, N, K, pitch(A), pitch(B),
                         pitch(C)),
              "gemm (bf16)");
    return;
  }
  if (A.kind == ElemKind::F32 && !workspace.is_none()) {
    ArrayArg ws = deviceArray(ctx, workspace, "workspace", 1);
    ctx.check(hcGemmF32Tensor(ctx.get(), A.data, B.data, C.data, ws.data,
                              size_t(ws.shape[0]) * size_t(ws.itemsize), M, N, K, pitch(A),
                              pitch(B), pitch(C)),
              "gemm (float32, tensor cores)");
    return;
  }
  ctx.check(hcGemmTiled(ctx.get(), A.data, B.data, C.data, M, N, K, pitch(A), pitch(B),
                        pitch(C), floatDType(A, "a")),
            "gemm");
}

size_t w8a16WorkspaceBytes(long long n, long long k) {
  return hcGemmW8A16WorkspaceBytes(n, k);
}

void gemmW8A16(Context &ctx, py::handle a, py::handle w, py::handle scale, py::handle out,
               py::object workspace) {
  ArrayArg A = deviceArray(ctx, a, "a", 2), W = deviceArray(ctx, w, "w", 2),
           S = deviceArray(ctx, scale, "scale", 1), C = deviceArray(ctx, out, "out", 2);
  if (A.kind != ElemKind::BF16 || C.kind != ElemKind::BF16)
    throw py::type_error("gemm_w8a16: a and out must be bfloat16");
  if (W.kind != ElemKind::I8)
    throw py::type_error(std::string("gemm_w8a16: w must be int8, got ") + hc::kindName(W.kind));
  if (S.kind != ElemKind::F32)
    throw py::type_error("gemm_w8a16: scale must be float32");
  long long M = A.shape[0], K = A.shape[1], N = W.shape[1];
  if (W.shape[0] != K || C.shape[0] != M || C.shape[1] != N || S.shape[0] != N)
    throw py::value_error("gemm_w8a16: shapes do not form [M,K] @ [K,N] * [N] -> [M,N]");
  if (N > 1 && S.strides[0] != 1)
    throw py::value_error("scale: must be contiguous");
  void *ws = nullptr;
  size_t wsBytes = 0;
  if (!workspace.is_none()) {
    ArrayArg Wk = hc::arrayFromPython(workspace);
    if (!Wk.onDevice)
      throw py::value_error("workspace: expected device memory");
    ws = Wk.data;
    wsBytes = size_t(Wk.itemsize);
    for (auto d : Wk.shape)
      wsBytes *= size_t(d);
  }
  ctx.check(hcGemmW8A16(ctx.get(), A.data, W.data, static_cast<const float *>(S.data), C.data,
                        ws, wsBytes, M, N, K, pitch(A), pitch(W), pitch(C)),
            "gemm_w8a16");
}

} // namespace

PYBIND11_MODULE(_dispatcher, m) {
  m.doc() = "Launch path of hc_b200: argument checking + precompiled sm_100a kernels";

  py::class_<Context>(m, "Context")
      .def(py::init<const std::string &>(), py::arg("device") = "cuda:0")
      .def("close", &Context::close)
      .def_readonly("device", &Context::description)
      .def_readonly("ordinal", &Context::ordinal)
      .def_property_readonly("stream",
                             [](Context &c) {
                               return reinterpret_cast<uintptr_t>(hcContextStream(c.get()));
                             })
      .def_property_readonly("launch_count",
                             [](Context &c) { return hcLaunchCount(c.get()); })
      .def("synchronize", [](Context &c) { c.check(hcSynchronize(c.get()), "synchronize"); })
      .def("kernel_status",
           [](Context &c) {
             int v = 0;
             c.check(hcKernelStatus(c.get(), &v), "kernel_status");
             return v;
           })
      .def("set_option", [](Context &c, const std::string &name, long long v) {
        c.check(hcSetOption(c.get(), name.c_str(), v), "set_option");
      })
      // Programs compiled at run time by this context (or loaded from the directory
      // of HC_B200_KERNEL_CACHE), and why the latest attempt failed.
      .def("specialised_programs",
           [](Context &c, bool fromDisk) { return hcSpecialisedPrograms(c.get(), fromDisk); },
           py::arg("from_disk") = false)
      .def_property_readonly("specialise_note", [](Context &c) {
        return std::string(hcSpecialiseNote(c.get()));
      });

  m.def("copy2d", &copy2d, py::arg("ctx"), py::arg("src"), py::arg("dst"));
  m.def("softmax_rows", &softmaxRows, py::arg("ctx"), py::arg("x"), py::arg("out"));
  m.def("reduce_rows", &reduceRows, py::arg("ctx"), py::arg("x"),
        py::arg("sum_out") = py::none(), py::arg("max_out") = py::none());
  m.def("reduce_all", &reduceAll, py::arg("ctx"), py::arg("a"), py::arg("result"));
  m.def("softmax_rows_peers", &softmaxRowsPeers, py::arg("ctx"), py::arg("x"), py::arg("bases"),
        py::arg("out_pitch"));
  m.def("gemm_bf16_peers", &gemmBf16Peers, py::arg("ctx"), py::arg("a"), py::arg("b"),
        py::arg("bases"), py::arg("out_pitch"));
  m.def("gemm_w8a16_peers", &gemmW8A16Peers, py::arg("ctx"), py::arg("a"), py::arg("w"),
        py::arg("scale"), py::arg("bases"), py::arg("out_pitch"), py::arg("workspace"));
  m.def("reduce_rows_peers", &reduceRowsPeers, py::arg("ctx"), py::arg("x"), py::arg("bases"),
        py::arg("max_offset"));
  m.def("softmax_rows_host", &softmaxRowsHost, py::arg("ctx"), py::arg("x"), py::arg("out"));
  m.def("reduce_rows_host", &reduceRowsHost, py::arg("ctx"), py::arg("x"),
        py::arg("sum_out") = py::none(), py::arg("max_out") = py::none());
  m.def("gemm_bf16_host", &gemmBf16Host, py::arg("ctx"), py::arg("a"), py::arg("b"),
        py::arg("out"));
  m.def("pairwise_distance", &pairwiseDistance, py::arg("ctx"), py::arg("a"), py::arg("b"),
        py::arg("out"));
  m.def("map_elements", &mapElements, py::arg("ctx"), py::arg("inputs"), py::arg("out"),
        py::arg("code"), py::arg("consts"));
  m.def("work_items", &workItems, py::arg("ctx"), py::arg("inputs"), py::arg("offsets"),
        py::arg("out"), py::arg("group"), py::arg("code"), py::arg("consts"), py::arg("guards"),
        py::arg("tiles"), py::arg("tile_fill") = 0.0);
  m.def("row_program", &rowProgram, py::arg("ctx"), py::arg("inputs"), py::arg("out"),
        py::arg("code"), py::arg("consts"));
  m.def("mapped_gemm", &mappedGemm, py::arg("ctx"), py::arg("x"), py::arg("x_tables"),
        py::arg("f"), py::arg("f_tables"), py::arg("out"), py::arg("out_tables"),
        py::arg("groups"), py::arg("tm"), py::arg("tn"), py::arg("k"));
  m.def("gemm", &gemm, py::arg("ctx"), py::arg("a"), py::arg("b"), py::arg("out"),
        py::arg("workspace") = py::none());
  m.def("gemm_f32_workspace_bytes", &gemmF32WorkspaceBytes, py::arg("m"), py::arg("n"),
        py::arg("k"));
  m.def("conv_f32_tensor", &convF32Tensor, py::arg("ctx"), py::arg("x"), py::arg("f"),
        py::arg("out"), py::arg("stride"), py::arg("workspace"));
  m.def("conv_f32_workspace_bytes", &convF32WorkspaceBytes, py::arg("n"), py::arg("c"),
        py::arg("h"), py::arg("w"), py::arg("nf"), py::arg("hf"), py::arg("wf"));
  m.def("gemm_w8a16", &gemmW8A16, py::arg("ctx"), py::arg("a"), py::arg("w"),
        py::arg("scale"), py::arg("out"), py::arg("workspace") = py::none());
  m.def("w8a16_workspace_bytes", &w8a16WorkspaceBytes, py::arg("n"), py::arg("k"));
  m.def("image_names", [] {
    std::vector<std::string> names;
    for (int i = 0; i < hcImageCount(); ++i)
      names.emplace_back(hcImageName(i));
    return names;
  });
}
