// Run-time specialisation of element-wise and row programs.
//
// The reference compiles every kernel body at its first call (Python -> MLIR ->
// GPU binary, python/hckernel/dispatcher.py:81-137 and the specialisation cache
// of python/cpp/native/DispatcherBase.cpp:250-256,542-585).  Here a body reaches
// the library as a short program for the accumulator machine (map_params.h).
// The interpreting kernels (map_elements.cu, row_program.cu) run any program at
// once; the bodies of fused_programs.h were turned into straight-line kernels
// when the library was built.  This file does the same for any other program
// the first time it is launched: the kernel sources that the ahead-of-time
// bodies are made from (map_fused.cu, row_fused.cu and their headers, embedded
// in this library as text) are compiled by NVRTC for the device at hand with
// the program's instruction words as template constants, the resulting image is
// loaded through olCreateModule, and its kernels are kept for the lifetime of
// the context under the program's words.  Results are bit for bit those of the
// interpreter, as for the ahead-of-time bodies (same templates).
//
// NVRTC is looked up at run time (dlopen): without it, or when a compilation
// fails, the program is interpreted and the reason is kept for hcSpecialiseNote.
// With the directory named by HC_B200_KERNEL_CACHE the compiled images are also
// kept on disk, under a hash of everything that went into them.
#include "context.hpp"
#include "../kernels/items_params.h"

#include "../kernels/map_params.h"

#include <algorithm>
#include <cinttypes>
#include <cstring>
#include <dlfcn.h>
#include <fstream>
#include <sstream>
#include <sys/stat.h>
#include <unistd.h>

// Kernel sources embedded next to the images (images_gen.S).
struct HcSourceText {
  const char *name;
  const char *begin;
  const char *end;
};
extern "C" const HcSourceText hc_b200_sources[];
extern "C" const int hc_b200_source_count;

namespace {

// The few NVRTC entry points used, resolved by name.
struct Nvrtc {
  using Program = struct _nvrtcProgram *;
  int (*createProgram)(Program *, const char *, const char *, int, const char *const *,
                       const char *const *) = nullptr;
  int (*compileProgram)(Program, int, const char *const *) = nullptr;
  int (*getCUBINSize)(Program, size_t *) = nullptr;
  int (*getCUBIN)(Program, char *) = nullptr;
  int (*getProgramLogSize)(Program, size_t *) = nullptr;
  int (*getProgramLog)(Program, char *) = nullptr;
  int (*destroyProgram)(Program *) = nullptr;
  int (*version)(int *, int *) = nullptr;
  const char *(*getErrorString)(int) = nullptr;
  void *lib = nullptr;
  std::string why; // why it could not be loaded

  bool load() {
    if (lib)
      return true;
    if (!why.empty())
      return false;
    std::vector<std::string> names;
    if (const char *env = getenv("HC_B200_NVRTC"))
      names.push_back(env);
    for (const char *n : {"libnvrtc.so.12", "libnvrtc.so", "/usr/local/cuda/lib64/libnvrtc.so.12",
                          "/usr/local/cuda/lib64/libnvrtc.so"})
      names.push_back(n);
    for (const std::string &n : names)
      if ((lib = dlopen(n.c_str(), RTLD_NOW | RTLD_LOCAL)))
        break;
    if (!lib) {
      why = "NVRTC not found (libnvrtc.so.12; HC_B200_NVRTC names another path)";
      return false;
    }
    auto bind = [&](auto &fn, const char *symbol) {
      fn = reinterpret_cast<std::decay_t<decltype(fn)>>(dlsym(lib, symbol));
      if (!fn && why.empty())
        why = std::string("NVRTC lacks ") + symbol;
    };
    bind(createProgram, "nvrtcCreateProgram");
    bind(compileProgram, "nvrtcCompileProgram");
    bind(getCUBINSize, "nvrtcGetCUBINSize");
    bind(getCUBIN, "nvrtcGetCUBIN");
    bind(getProgramLogSize, "nvrtcGetProgramLogSize");
    bind(getProgramLog, "nvrtcGetProgramLog");
    bind(destroyProgram, "nvrtcDestroyProgram");
    bind(version, "nvrtcVersion");
    bind(getErrorString, "nvrtcGetErrorString");
    if (!why.empty()) {
      dlclose(lib);
      lib = nullptr;
      return false;
    }
    return true;
  }
};

Nvrtc &nvrtc() {
  static Nvrtc instance; // like cuInit in the backend: one per process, no lock
  return instance;
}

// What the kernel sources include from the system, as far as they use it: NVRTC
// has no C library headers, and declares the device math functions itself.
const char kStdint[] = "#pragma once\n"
                       "typedef signed char int8_t; typedef unsigned char uint8_t;\n"
                       "typedef short int16_t; typedef unsigned short uint16_t;\n"
                       "typedef int int32_t; typedef unsigned int uint32_t;\n"
                       "typedef long int64_t; typedef unsigned long uint64_t;\n";
const char kMath[] = "#pragma once\n#define INFINITY __int_as_float(0x7f800000)\n";
const char kTypeTraits[] =
    "#pragma once\n"
    "namespace std {\n"
    "template <typename T> struct make_unsigned { using type = T; };\n"
    "template <> struct make_unsigned<int> { using type = unsigned int; };\n"
    "template <> struct make_unsigned<long> { using type = unsigned long; };\n"
    "template <> struct make_unsigned<long long> { using type = unsigned long long; };\n"
    "template <typename A, typename B> struct is_same { static constexpr bool value = false; };\n"
    "template <typename A> struct is_same<A, A> { static constexpr bool value = true; };\n"
    "}\n";

const HcSourceText *embedded(const char *name) {
  for (int i = 0; i < hc_b200_source_count; ++i)
    if (std::strcmp(hc_b200_sources[i].name, name) == 0)
      return &hc_b200_sources[i];
  return nullptr;
}

uint64_t fnv1a(uint64_t h, const void *data, size_t len) {
  const auto *p = static_cast<const unsigned char *>(data);
  for (size_t i = 0; i < len; ++i)
    h = (h ^ p[i]) * 0x100000001b3ull;
  return h;
}

} // namespace

struct HcSpecialiser {
  struct Entry {
    std::string tag;  // part of the kernel names: hc_map_fused_<tag>_f32_v4 ...
    OlModule module = nullptr;
    bool failed = false;
  };
  std::map<std::string, Entry> entries; // by kind, element type and instruction words
  std::string note;
  long long compiled = 0, fromDisk = 0;
};

void hcReleaseSpecialiser(HcContextImpl *c) {
  if (!c->specialiser)
    return;
  for (auto &kv : c->specialiser->entries)
    if (kv.second.module)
      olReleaseModule(kv.second.module);
  delete c->specialiser;
  c->specialiser = nullptr;
}

const char *hcSpecialiserNote(HcContextImpl *c) {
  return c->specialiser ? c->specialiser->note.c_str() : "";
}

long long hcSpecialiserCount(HcContextImpl *c, int which) {
  if (!c->specialiser)
    return 0;
  return which == 0 ? c->specialiser->compiled : c->specialiser->fromDisk;
}

// What the straight-line kernels cover: element-wise programs of any operation
// on the four element types; row programs of the operations up to `set` on
// floats (the later operators are not allowed in row programs at all).
bool hcSpecialisable(const HcMapProgramDev &p, bool row, int dtype) {
  const bool floating = dtype == HC_F32 || dtype == HC_F64;
  if (!floating && (row || (dtype != HC_I32 && dtype != HC_I64)))
    return false;
  for (int pc = 0; pc < p.nInstr; ++pc) {
    const uint32_t op = p.code[pc] & 0x7fu;
    if (row ? op >= HC_MAP_FLOORDIV
            : op >= HC_MAP_OP_COUNT || op == HC_MAP_RSUM || op == HC_MAP_RMAX || op == HC_MAP_SET)
      return false;
  }
  return true;
}

namespace {

// 0 float32, 1 float64, 2 int32, 3 int64: the value of HC_FUSED_ONLY.
int typeIndex(int dtype) {
  return dtype == HC_F32 ? 0 : dtype == HC_F64 ? 1 : dtype == HC_I32 ? 2 : 3;
}
const char *const kTypeNames[] = {"f32", "f64", "i32", "i64"};

// What is compiled: an element-wise program, a row program, a work-item program.
enum Kind { kMap = 0, kRow = 1, kItem = 2 };
struct KindText {
  const char *name;     // part of the kernel and structure names
  const char *source;   // the embedded translation unit
  const char *listName; // the list macro of the generated header
};
const KindText kKinds[] = {{"map", "map_fused.cu", "MAP"},
                           {"row", "row_fused.cu", "ROW"},
                           {"item", "work_items.cu", "ITEM"}};

std::string programKey(Kind kind, int dtype, int nInputs, const uint32_t *code, int nInstr) {
  std::string key(kKinds[kind].name);
  key += kTypeNames[typeIndex(dtype)];
  key += char('0' + nInputs);
  key.append(reinterpret_cast<const char *>(code), size_t(nInstr) * sizeof(uint32_t));
  return key;
}

// The device image with the kernels of program `p` for compute capability
// major.minor, from the directory of HC_B200_KERNEL_CACHE or from NVRTC.  `tag`
// is the part of the kernel names that stands for the program.  False, with the
// reason in `why`, when there is no way to get one.
bool buildImage(Kind what, int dtype, int nInputs, const uint32_t *code, int nInstr,
                long long ccMajor, long long ccMinor, std::string &image, std::string &tag,
                bool &fromDisk, std::string &why) {
  const char *kind = kKinds[what].name;
  const HcSourceText *main = embedded(kKinds[what].source);
  const char *headerNames[] = {"fused_machine.cuh", "map_machine.cuh", "map_params.h",
                               "items_params.h"};
  if (!main) {
    why = "the kernel sources are not embedded in this library";
    return false;
  }
  const std::string key = programKey(what, dtype, nInputs, code, nInstr);
  char tagText[32];
  std::snprintf(tagText, sizeof tagText, "j%016" PRIx64,
                fnv1a(0xcbf29ce484222325ull, key.data(), key.size()));
  tag = tagText;

  // The program as the header the kernel source includes.
  std::ostringstream programs;
  programs << "#pragma once\n#include <stdint.h>\nnamespace hcfused {\nstruct " << kind << "_" << tag
           << " {\n  static constexpr int nin = " << nInputs << ", n = " << nInstr
           << ";\n  static constexpr uint32_t code[" << nInstr << "] = {";
  for (int pc = 0; pc < nInstr; ++pc)
    programs << (pc ? ", " : "") << code[pc] << "u";
  programs << "};\n};\n}\n#define HC_FUSED_" << kKinds[what].listName << "_LIST(X) X(" << tag
           << ")\n";

  std::vector<std::string> texts = {programs.str(), kStdint, kMath, kTypeTraits};
  std::vector<const char *> names = {"fused_programs.h", "stdint.h", "math.h", "type_traits"};
  for (const char *h : headerNames) {
    const HcSourceText *t = embedded(h);
    if (!t) {
      why = std::string("the kernel source ") + h + " is not embedded in this library";
      return false;
    }
    texts.emplace_back(t->begin, t->end);
    names.push_back(h);
  }
  const std::string mainText(main->begin, main->end);
  char arch[40];
  // The arch-specific suffix exists from sm_90a on.
  std::snprintf(arch, sizeof arch, "--gpu-architecture=sm_%lld%lld%s", ccMajor, ccMinor,
                ccMajor >= 9 ? "a" : "");
  // One element type per image; the work-item source compiles its fixed-program
  // form when told so, for one class of work-group sizes (nInputs: 1 = the wide
  // form for small groups).
  char only[32];
  std::snprintf(only, sizeof only, "-DHC_FUSED_ONLY=%d", typeIndex(dtype));
  const char *options[] = {arch, "--std=c++17", "-lineinfo", only,
                           what == kItem ? "-DHC_ITEM_FIXED_PROGRAM=1" : "-DHC_UNUSED=1",
                           what == kItem && nInputs == 1 ? "-DHC_ITEM_WIDE=1" : "-DHC_UNUSED2=1"};
  const int optionCount = 6;

  // On disk, under a hash of all the text and the options.
  std::string cachePath;
  if (const char *dir = getenv("HC_B200_KERNEL_CACHE")) {
    uint64_t h = fnv1a(0xcbf29ce484222325ull, mainText.data(), mainText.size());
    for (const std::string &t : texts)
      h = fnv1a(h, t.data(), t.size());
    for (const char *o : options)
      h = fnv1a(h, o, std::strlen(o));
    char file[64];
    std::snprintf(file, sizeof file, "/hc-%s-%016" PRIx64 ".cubin", kind, h);
    cachePath = std::string(dir) + file;
    std::ifstream in(cachePath, std::ios::binary);
    if (in) {
      std::ostringstream all;
      all << in.rdbuf();
      image = all.str();
      if (!image.empty()) {
        fromDisk = true;
        return true;
      }
    }
  }
  fromDisk = false;
  Nvrtc &rtc = nvrtc();
  if (!rtc.load()) {
    why = rtc.why;
    return false;
  }
  std::vector<const char *> headerTexts;
  for (const std::string &t : texts)
    headerTexts.push_back(t.c_str());
  Nvrtc::Program prog = nullptr;
  int rc = rtc.createProgram(&prog, mainText.c_str(), kKinds[what].source, int(names.size()),
                             headerTexts.data(), names.data());
  if (rc != 0) {
    why = std::string("nvrtcCreateProgram: ") + rtc.getErrorString(rc);
    return false;
  }
  rc = rtc.compileProgram(prog, optionCount, options);
  if (rc != 0) {
    size_t n = 0;
    rtc.getProgramLogSize(prog, &n);
    std::string log(n, '\0');
    if (n)
      rtc.getProgramLog(prog, &log[0]);
    rtc.destroyProgram(&prog);
    why = std::string("nvrtcCompileProgram: ") + rtc.getErrorString(rc) + "\n" + log;
    return false;
  }
  size_t n = 0;
  if (rtc.getCUBINSize(prog, &n) != 0 || n == 0) {
    rtc.destroyProgram(&prog);
    why = "NVRTC produced no device image";
    return false;
  }
  image.resize(n);
  rtc.getCUBIN(prog, &image[0]);
  rtc.destroyProgram(&prog);
  if (!cachePath.empty()) {
    // Written under another name first, so that a reader never sees half a file.
    const std::string tmp = cachePath + "." + std::to_string(getpid());
    std::ofstream out(tmp, std::ios::binary);
    if (out && out.write(image.data(), std::streamsize(image.size())) && (out.close(), true))
      rename(tmp.c_str(), cachePath.c_str());
  }
  return true;
}

} // namespace

// The tag of the kernels compiled for program `p` (`row`: a row program, else
// element-wise; `f64`: the element type), compiling them first if this context
// has not seen the program yet.  nullptr when that is not possible; the reason
// is then in hcSpecialiserNote().
const char *hcSpecialise(HcContextImpl *c, bool row, int dtype, const HcMapProgramDev &p) {
  if (!c->specialiser)
    c->specialiser = new HcSpecialiser;
  HcSpecialiser &s = *c->specialiser;
  const Kind what = row ? kRow : kMap;
  const std::string key = programKey(what, dtype, p.nInputs, p.code, p.nInstr);
  auto found = s.entries.find(key);
  if (found != s.entries.end())
    return found->second.failed ? nullptr : found->second.tag.c_str();
  HcSpecialiser::Entry &entry = s.entries[key];
  entry.failed = true; // until the kernels are there
  std::string image, tag;
  bool fromDisk = false;
  if (!buildImage(what, dtype, p.nInputs, p.code, p.nInstr, c->ccMajor, c->ccMinor, image, tag,
                  fromDisk, s.note))
    return nullptr;
  OlModule module = olCreateModule(c->device, image.data(), image.size());
  if (!module) {
    s.note = "olCreateModule failed for a specialised image: " + c->lastError;
    return nullptr;
  }
  // Every kernel of the image, under its name, beside those of the embedded images.
  static const char *const mapVariants[] = {"f32_v4", "f32_v1", "f64_v2", "f64_v1",
                                            "i32_v4", "i32_v1", "i64_v2", "i64_v1"};
  static const char *const rowVariants[] = {"f32_held_t64", "f32_held_t128", "f32_v4",
                                            "f32_v1",       "f64_v2",        "f64_v1"};
  const char *const *variants = row ? rowVariants : mapVariants;
  const int count = row ? 6 : 8;
  for (int i = 0; i < count; ++i) {
    if (std::strncmp(variants[i], kTypeNames[typeIndex(dtype)], 3) != 0)
      continue;
    char name[96];
    std::snprintf(name, sizeof name, "hc_%s_fused_%s_%s", row ? "row" : "map", tag.c_str(),
                  variants[i]);
    OlKernel k = olGetKernel(module, name);
    if (!k) {
      olReleaseModule(module);
      s.note = std::string("a specialised image lacks ") + name + ": " + c->lastError;
      return nullptr;
    }
    c->kernels[name] = k;
  }
  entry.tag = tag;
  entry.module = module;
  entry.failed = false;
  ++(fromDisk ? s.fromDisk : s.compiled);
  return entry.tag.c_str();
}

// The same for a work-item program (hcWorkItems): the tag of the kernel
// hc_work_items_fused_<tag>_{f32,f64}, or nullptr.
const char *hcSpecialiseItems(HcContextImpl *c, int dtype, const uint32_t *code, int nInstr,
                              bool wide) {
  if (!c->specialiser)
    c->specialiser = new HcSpecialiser;
  HcSpecialiser &s = *c->specialiser;
  const std::string key = programKey(kItem, dtype, wide ? 1 : 0, code, nInstr);
  auto found = s.entries.find(key);
  if (found != s.entries.end())
    return found->second.failed ? nullptr : found->second.tag.c_str();
  HcSpecialiser::Entry &entry = s.entries[key];
  entry.failed = true;
  std::string image, tag;
  bool fromDisk = false;
  if (!buildImage(kItem, dtype, wide ? 1 : 0, code, nInstr, c->ccMajor, c->ccMinor, image, tag,
                  fromDisk, s.note))
    return nullptr;
  OlModule module = olCreateModule(c->device, image.data(), image.size());
  if (!module) {
    s.note = "olCreateModule failed for a specialised image: " + c->lastError;
    return nullptr;
  }
  char name[96];
  std::snprintf(name, sizeof name, "hc_work_items_fused_%s_%s", tag.c_str(),
                kTypeNames[typeIndex(dtype)]);
  OlKernel k = olGetKernel(module, name);
  if (!k) {
    olReleaseModule(module);
    s.note = std::string("a specialised image lacks ") + name + ": " + c->lastError;
    return nullptr;
  }
  c->kernels[name] = k;
  entry.tag = tag;
  entry.module = module;
  entry.failed = false;
  ++(fromDisk ? s.fromDisk : s.compiled);
  return entry.tag.c_str();
}

// Compiles without a context or a GPU: the image for compute capability
// major.minor, copied to `image` as far as `capacity` allows.
extern "C" HC_B200_API long long hcSpecialiseCompile(const HcMapProgram *program, int rowProgram,
                                                     int dtype, int ccMajor, int ccMinor,
                                                     void *image, size_t capacity, char *message,
                                                     size_t messageCapacity) {
  auto say = [&](const std::string &text) {
    if (message && messageCapacity)
      std::snprintf(message, messageCapacity, "%s", text.c_str());
    return -1ll;
  };
  if (!program)
    return say("hcSpecialiseCompile: null program");
  HcMapProgramDev p;
  std::memcpy(&p, program, sizeof p);
  if (p.nInstr < 1 || p.nInstr > HC_MAP_MAX_INSTR || p.nInputs < 0 ||
      p.nInputs > HC_MAP_MAX_INPUTS)
    return say("hcSpecialiseCompile: the program has no valid size");
  if (!hcSpecialisable(p, rowProgram != 0, dtype))
    return say("hcSpecialiseCompile: element-wise programs on float32, float64, int32 or int64; "
               "row programs of the operations up to `set` on float32 or float64");
  std::string bytes, tag, why;
  bool fromDisk = false;
  if (!buildImage(rowProgram != 0 ? kRow : kMap, dtype, p.nInputs, p.code, p.nInstr, ccMajor,
                  ccMinor, bytes, tag, fromDisk, why))
    return say(why);
  if (image && capacity)
    std::memcpy(image, bytes.data(), std::min(capacity, bytes.size()));
  say(tag);
  return (long long)bytes.size();
}

// The same for a work-item program: `code` holds nInstr instruction words of
// hcWorkItems' program; dtype HC_F32 or HC_F64; groupThreads the work-group size
// the kernel is to serve (one kernel up to HC_ITEM_WIDE_THREADS, another beyond).
extern "C" HC_B200_API long long hcSpecialiseCompileItems(const unsigned *code, int nInstr,
                                                          int dtype, int groupThreads,
                                                          int ccMajor, int ccMinor,
                                                          void *image, size_t capacity,
                                                          char *message, size_t messageCapacity) {
  auto say = [&](const std::string &text) {
    if (message && messageCapacity)
      std::snprintf(message, messageCapacity, "%s", text.c_str());
    return -1ll;
  };
  if (!code || nInstr < 1 || nInstr > HC_ITEM_MAX_INSTR)
    return say("hcSpecialiseCompileItems: the program has no valid size");
  if (dtype != HC_F32 && dtype != HC_F64)
    return say("hcSpecialiseCompileItems: work-item programs run on float32 or float64");
  if (groupThreads < 1 || groupThreads > 1024)
    return say("hcSpecialiseCompileItems: work-groups have 1 to 1024 work-items");
  std::string bytes, tag, why;
  bool fromDisk = false;
  if (!buildImage(kItem, dtype, groupThreads <= HC_ITEM_WIDE_THREADS ? 1 : 0, code, nInstr,
                  ccMajor, ccMinor, bytes, tag, fromDisk, why))
    return say(why);
  if (image && capacity)
    std::memcpy(image, bytes.data(), std::min(capacity, bytes.size()));
  say(tag);
  return (long long)bytes.size();
}
