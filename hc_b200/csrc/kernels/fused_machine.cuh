// The accumulator machine of map_machine.cuh with the program known at compile
// time: every instruction word is a template constant, so a program becomes
// straight-line code on registers - no decoding, no operand selection, no
// copies between the accumulator and the inputs.  The operations are the same,
// in the same order, each rounded on its own (the *_rn intrinsics are never
// contracted into fused multiply-adds), so a precompiled program gives bit for
// bit what the interpreter gives for the same instruction words.
//
// A program type P provides `nin`, `n` and `code[n]` (fused_programs.h).
#pragma once

#include "map_machine.cuh"

namespace hcfused {

// Integers: the interpreter's own wrapping arithmetic (nothing to contract).
template <typename T> struct Arith {
  static __device__ __forceinline__ T add(T a, T b) { return hcmap::addOf(a, b); }
  static __device__ __forceinline__ T sub(T a, T b) { return hcmap::subOf(a, b); }
  static __device__ __forceinline__ T mul(T a, T b) { return hcmap::mulOf(a, b); }
  static __device__ __forceinline__ T div(T a, T b) { return hcmap::Num<T>::div(a, b); }
  static __device__ __forceinline__ T sqrt(T a) { return hcmap::Num<T>::sqrtOf(a); }
  static __device__ __forceinline__ T exp(T a) { return hcmap::Num<T>::exp(a); }
  static __device__ __forceinline__ T log(T a) { return hcmap::Num<T>::log(a); }
  static __device__ __forceinline__ T max(T a, T b) { return hcmap::maxOf(a, b); }
  static __device__ __forceinline__ T min(T a, T b) { return hcmap::minOf(a, b); }
};
template <> struct Arith<float> {
  static __device__ __forceinline__ float add(float a, float b) { return __fadd_rn(a, b); }
  static __device__ __forceinline__ float sub(float a, float b) { return __fsub_rn(a, b); }
  static __device__ __forceinline__ float mul(float a, float b) { return __fmul_rn(a, b); }
  static __device__ __forceinline__ float div(float a, float b) { return __fdiv_rn(a, b); }
  static __device__ __forceinline__ float sqrt(float a) { return __fsqrt_rn(a); }
  static __device__ __forceinline__ float exp(float a) { return expf(a); }
  static __device__ __forceinline__ float log(float a) { return logf(a); }
  // As the interpreter: NaN if either operand is NaN, the first operand on a tie.
  static __device__ __forceinline__ float max(float a, float b) { return hcmap::maxOf(a, b); }
  static __device__ __forceinline__ float min(float a, float b) { return hcmap::minOf(a, b); }
};
template <> struct Arith<double> {
  static __device__ __forceinline__ double add(double a, double b) { return __dadd_rn(a, b); }
  static __device__ __forceinline__ double sub(double a, double b) { return __dsub_rn(a, b); }
  static __device__ __forceinline__ double mul(double a, double b) { return __dmul_rn(a, b); }
  static __device__ __forceinline__ double div(double a, double b) { return __ddiv_rn(a, b); }
  static __device__ __forceinline__ double sqrt(double a) { return __dsqrt_rn(a); }
  static __device__ __forceinline__ double exp(double a) { return ::exp(a); }
  static __device__ __forceinline__ double log(double a) { return ::log(a); }
  static __device__ __forceinline__ double max(double a, double b) { return hcmap::maxOf(a, b); }
  static __device__ __forceinline__ double min(double a, double b) { return hcmap::minOf(a, b); }
};

template <typename T, uint32_t OP> __device__ __forceinline__ T binaryOp(T a, T b) {
  if constexpr (OP == HC_MAP_LOAD) return b;
  else if constexpr (OP == HC_MAP_ADD) return Arith<T>::add(a, b);
  else if constexpr (OP == HC_MAP_SUB) return Arith<T>::sub(a, b);
  else if constexpr (OP == HC_MAP_RSUB) return Arith<T>::sub(b, a);
  else if constexpr (OP == HC_MAP_MUL) return Arith<T>::mul(a, b);
  else if constexpr (OP == HC_MAP_DIV) return Arith<T>::div(a, b);
  else if constexpr (OP == HC_MAP_RDIV) return Arith<T>::div(b, a);
  else if constexpr (OP == HC_MAP_MAX) return Arith<T>::max(a, b);
  else if constexpr (OP == HC_MAP_MIN) return Arith<T>::min(a, b);
  // The later operators, as the extended interpreter computes them.
  else if constexpr (OP == HC_MAP_LT) return T(a < b);
  else if constexpr (OP == HC_MAP_LE) return T(a <= b);
  else if constexpr (OP == HC_MAP_EQ) return T(a == b);
  else if constexpr (OP == HC_MAP_NE) return T(a != b);
  else if constexpr (OP == HC_MAP_GE) return T(a >= b);
  else if constexpr (OP == HC_MAP_GT) return T(a > b);
  else if constexpr (OP == HC_MAP_AND) return hcmap::Num<T>::bitAnd(a, b);
  else if constexpr (OP == HC_MAP_OR) return hcmap::Num<T>::bitOr(a, b);
  else if constexpr (OP == HC_MAP_XOR) return hcmap::Num<T>::bitXor(a, b);
  else if constexpr (OP == HC_MAP_SHL) return hcmap::Num<T>::shl(a, b);
  else if constexpr (OP == HC_MAP_SHR) return hcmap::Num<T>::shr(a, b);
  else if constexpr (OP == HC_MAP_RSHL) return hcmap::Num<T>::shl(b, a);
  else {
    static_assert(OP == HC_MAP_RSHR, "not an operation of two operands on registers");
    return hcmap::Num<T>::shr(b, a);
  }
}

template <typename T, uint32_t OP> __device__ __forceinline__ T unaryOp(T a) {
  if constexpr (OP == HC_MAP_NEG) return hcmap::negOf(a);
  // As the interpreter writes it: -0 becomes +0, a NaN keeps its bits.
  else if constexpr (OP == HC_MAP_ABS) return hcmap::Num<T>::absOf(a);
  else if constexpr (OP == HC_MAP_EXP) return Arith<T>::exp(a);
  else if constexpr (OP == HC_MAP_SQRT) return Arith<T>::sqrt(a);
  else if constexpr (OP == HC_MAP_INV) return hcmap::Num<T>::inv(a);
  else {
    static_assert(OP == HC_MAP_LOG, "not an operation of one operand");
    return Arith<T>::log(a);
  }
}

// What a thread holds while it runs a program on W elements.
template <typename T, int W, int NIN> struct Frame {
  T x[NIN > 0 ? NIN : 1][W];  // the inputs (a program may have none: it computes from indices)
  T t[3][W];    // the temporaries (only those a program saves to become registers)
  T s[4];       // row scalars
  uint32_t ok = ~0u;                   // validity bits of the accumulator's elements
  uint32_t okT[3] = {~0u, ~0u, ~0u};   // ... and of the parked values
};

// Clears the validity bit of the elements whose division numpy.ma would mask
// (map_machine.cuh: Num<T>::divides); MASKED is false for row programs, which do
// not track validity, and then nothing is generated.
template <typename T, uint32_t OP, bool MASKED>
__device__ __forceinline__ void noteDivision(uint32_t &ok, int i, T a, T b) {
  if constexpr (MASKED && (OP == HC_MAP_DIV || OP == HC_MAP_RDIV)) {
    if (!(OP == HC_MAP_DIV ? hcmap::Num<T>::divides(a, b) : hcmap::Num<T>::divides(b, a)))
      ok &= ~(1u << i);
  }
}

// acc = acc OP b for element i, with the validity bit kept up to date.  Floor
// division, remainder and power go through the interpreter's out-of-line
// routine (map_machine.cuh: rareBinary), which also says whether numpy.ma would
// mask the result.
template <typename T, uint32_t OP, bool MASKED>
__device__ __forceinline__ void apply(uint32_t &ok, int i, T &acc, T b) {
  if constexpr (OP >= HC_MAP_FLOORDIV && OP <= HC_MAP_RPOW) {
    bool valid;
    acc = hcmap::rareBinary<T>(OP, acc, b, valid);
    if (MASKED && !valid)
      ok &= ~(1u << i);
  } else {
    noteDivision<T, OP, MASKED>(ok, i, acc, b);
    acc = binaryOp<T, OP>(acc, b);
  }
}

// First instruction at or after `pc` that is not part of a uniform prologue.
template <typename P> __host__ __device__ constexpr int afterUniform(int pc) {
  while (pc < P::n && (P::code[pc] & HC_MAP_UNIFORM))
    ++pc;
  return pc;
}
// Where the pass that starts at `pc` ends: at its reduction instruction, or at
// the end of the program.
template <typename P> __host__ __device__ constexpr int passEnd(int pc) {
  while (pc < P::n && (P::code[pc] & 0xffu) != HC_MAP_RSUM && (P::code[pc] & 0xffu) != HC_MAP_RMAX)
    ++pc;
  return pc;
}
template <typename P> __host__ __device__ constexpr bool usesIndices() {
  for (int pc = 0; pc < P::n; ++pc) {
    const uint32_t op = P::code[pc] & 0xffu, src = P::code[pc] >> 8;
    if (hcMapIsBinary(op) && (src == HC_MAP_SRC_ROW || src == HC_MAP_SRC_COL))
      return true;
  }
  return false;
}

// Instructions [PC, END) on the W elements of a thread.  `row` / `packet` say
// where they sit (element i is in packet `packet + (i / V) * STRIDE`, position
// i % V), for programs that use the element indices.
template <typename T, int W, int V, int NIN, typename P, int PC, int END, int STRIDE,
          bool MASKED = false>
__device__ __forceinline__ void run(const HcMapProgramDev &p, Frame<T, W, NIN> &f, T (&acc)[W],
                                    long long row, long long packet) {
  if constexpr (PC < END) {
    constexpr uint32_t ins = P::code[PC], op = ins & 0xffu, src = ins >> 8;
    if constexpr (MASKED && op == HC_MAP_LOAD)
      f.ok = ~0u; // a fresh value (a parked one brings its own bits, below)
    if constexpr (hcMapIsBinary(op)) {
      if constexpr (src >= HC_MAP_SRC_SCALAR) {
        const T one = f.s[src - HC_MAP_SRC_SCALAR];
#pragma unroll
        for (int i = 0; i < W; ++i) {
          apply<T, op, MASKED>(f.ok, i, acc[i], one);
        }
      } else if constexpr (src == HC_MAP_SRC_COL) {
#pragma unroll
        for (int i = 0; i < W; ++i) {
          const T col = T((packet + (long long)(i / V) * STRIDE) * V + i % V);
          apply<T, op, MASKED>(f.ok, i, acc[i], col);
        }
      } else if constexpr (src == HC_MAP_SRC_ROW) {
        const T one = T(row);
#pragma unroll
        for (int i = 0; i < W; ++i) {
          apply<T, op, MASKED>(f.ok, i, acc[i], one);
        }
      } else if constexpr (src >= HC_MAP_SRC_CONST) {
        const T one = T(p.consts[src - HC_MAP_SRC_CONST]);
#pragma unroll
        for (int i = 0; i < W; ++i) {
          apply<T, op, MASKED>(f.ok, i, acc[i], one);
        }
      } else if constexpr (src >= HC_MAP_SRC_TEMP) {
        if constexpr (MASKED)
          f.ok = op == HC_MAP_LOAD ? f.okT[src - HC_MAP_SRC_TEMP]
                                   : f.ok & f.okT[src - HC_MAP_SRC_TEMP];
#pragma unroll
        for (int i = 0; i < W; ++i) {
          apply<T, op, MASKED>(f.ok, i, acc[i], f.t[src - HC_MAP_SRC_TEMP][i]);
        }
      } else {
        static_assert(src < uint32_t(NIN), "the program reads an input the kernel does not load");
#pragma unroll
        for (int i = 0; i < W; ++i) {
          apply<T, op, MASKED>(f.ok, i, acc[i], f.x[src][i]);
        }
      }
    } else if constexpr (op >= HC_MAP_SAVE0 && op <= HC_MAP_SAVE2) {
#pragma unroll
      for (int i = 0; i < W; ++i)
        f.t[op - HC_MAP_SAVE0][i] = acc[i];
      if constexpr (MASKED)
        f.okT[op - HC_MAP_SAVE0] = f.ok;
    } else {
#pragma unroll
      for (int i = 0; i < W; ++i)
        acc[i] = unaryOp<T, op>(acc[i]);
    }
    run<T, W, V, NIN, P, PC + 1, END, STRIDE, MASKED>(p, f, acc, row, packet);
  }
}

// The uniform prologue that starts at PC: one value per row, from constants
// and row scalars, ending in `set` instructions that write row scalars.
template <typename T, typename P, int PC>
__device__ __forceinline__ void runUniform(const HcMapProgramDev &p, T (&s)[4], T one) {
  if constexpr (PC < P::n && (P::code[PC < P::n ? PC : 0] & HC_MAP_UNIFORM) != 0) {
    constexpr uint32_t ins = P::code[PC], op = ins & 0x7fu, src = ins >> 8;
    if constexpr (op == HC_MAP_SET) {
      s[src] = one;
    } else if constexpr (op <= HC_MAP_MIN) {
      T b;
      if constexpr (src >= HC_MAP_SRC_SCALAR)
        b = s[src - HC_MAP_SRC_SCALAR];
      else
        b = T(p.consts[src - HC_MAP_SRC_CONST]);
      one = binaryOp<T, op>(one, b);
    } else {
      one = unaryOp<T, op>(one);
    }
    runUniform<T, P, PC + 1>(p, s, one);
  }
}

} // namespace hcfused
