// The expression machine shared by the element-wise kernel (map_elements.cu)
// and the row-program kernel (row_program.cu): one accumulator, three
// temporaries, up to four input arrays, eight constants (map_params.h).  A
// thread interprets the program on the W elements it holds in registers: one
// decode and one (uniform) branch per instruction, then W independent
// operations.  Operations are never contracted into FMAs, so + - * / and sqrt
// are the correctly rounded results NumPy gives.
//
// Element types: float, double, and (element-wise kernel only) int32 / int64,
// whose arithmetic wraps like NumPy's.  Besides the values a thread carries one
// validity bit per element: the division-like operations clear it where
// NumPy's masked arrays mask the element (the reference's tiles are numpy.ma
// arrays, python/hckernel/kernel_api.py:106-155): a zero divisor for / // %,
// a result that is not finite for **.  Invalid elements are not stored, like
// the reference's masked store (kernel_api.py:338-340).
#pragma once

#include "map_params.h"

#include <math.h>
#include <stdint.h>

#include <type_traits>

namespace hcmap {

constexpr int THREADS = 256;

template <typename T> __device__ __forceinline__ T expOf(T v);
template <> __device__ __forceinline__ float expOf<float>(float v) { return expf(v); }
template <> __device__ __forceinline__ double expOf<double>(double v) { return exp(v); }
template <typename T> __device__ __forceinline__ T logOf(T v);
template <> __device__ __forceinline__ float logOf<float>(float v) { return logf(v); }
template <> __device__ __forceinline__ double logOf<double>(double v) { return log(v); }

// NumPy's maximum/minimum: NaN if either operand is NaN; on a tie (+0 against
// -0) the second operand, which is what NumPy's vectorised loops return.
template <typename T> __device__ __forceinline__ T maxOf(T a, T b) {
  return (a > b || a != a) ? a : b;
}
template <typename T> __device__ __forceinline__ T minOf(T a, T b) {
  return (a < b || a != a) ? a : b;
}

// Arithmetic of one element type.  `divides(a, b)` is false where numpy.ma masks
// a / b, a // b and a % b (its _DomainSafeDivide: |a| * tiny >= |b|, with tiny
// the smallest normal double - for float32 and integers that is b == 0).
// Floor division and remainder of floats follow NumPy's npy_divmod step by
// step (fmod, quotient of the difference, Python's sign convention, the
// quotient snapped to the nearest integer), so the results are bit for bit
// NumPy's.
template <typename T> struct Num;

template <typename F> struct FloatNum {
  static constexpr bool isFloat = true;
  static __device__ __forceinline__ F fmodOf(float a, float b) { return fmodf(a, b); }
  static __device__ __forceinline__ F fmodOf(double a, double b) { return fmod(a, b); }
  static __device__ __forceinline__ F floorOf(float a) { return floorf(a); }
  static __device__ __forceinline__ F floorOf(double a) { return floor(a); }
  static __device__ __forceinline__ F signOf(F magnitude, float sign) {
    return copysignf(magnitude, sign);
  }
  static __device__ __forceinline__ F signOf(F magnitude, double sign) {
    return copysign(magnitude, sign);
  }
  // Quotient and remainder of NumPy's npy_divmod for b != 0.
  static __device__ __forceinline__ void divmod(F a, F b, F &quotient, F &remainder) {
    F mod = fmodOf(a, b);
    F div = (a - mod) / b;
    if (mod != F(0)) {
      if ((b < F(0)) != (mod < F(0))) {
        mod = mod + b;
        div = div - F(1);
      }
    } else {
      mod = signOf(F(0), b);
    }
    F floordiv;
    if (div != F(0)) {
      floordiv = floorOf(div);
      if (div - floordiv > F(0.5))
        floordiv = floordiv + F(1);
    } else {
      floordiv = signOf(F(0), a / b);
    }
    quotient = floordiv;
    remainder = mod;
  }
  static __device__ __forceinline__ F floordiv(F a, F b) {
    if (b == F(0))
      return a / b;
    F q, r;
    divmod(a, b, q, r);
    return q;
  }
  static __device__ __forceinline__ F mod(F a, F b) {
    if (b == F(0))
      return fmodOf(a, b);
    F q, r;
    divmod(a, b, q, r);
    return r;
  }
  static __device__ __forceinline__ bool finite(F a) { return isfinite(a); }
  static __device__ __forceinline__ F bitAnd(F a, F b) { return F(a != F(0) && b != F(0)); }
  static __device__ __forceinline__ F bitOr(F a, F b) { return F(a != F(0) || b != F(0)); }
  static __device__ __forceinline__ F bitXor(F a, F b) { return F((a != F(0)) != (b != F(0))); }
  static __device__ __forceinline__ F shl(F a, F) { return a; } // refused by the host
  static __device__ __forceinline__ F shr(F a, F) { return a; }
  static __device__ __forceinline__ F inv(F a) { return F(a == F(0)); }
  static __device__ __forceinline__ F absOf(F a) { return a < F(0) ? -a : (a == F(0) ? F(0) : a); }
  static __device__ __forceinline__ F div(F a, F b) { return a / b; }
  static __device__ __forceinline__ F sqrtOf(F a) { return sqrt(a); }
  static __device__ __forceinline__ F exp(F a) { return expOf(a); }
  static __device__ __forceinline__ F log(F a) { return logOf(a); }
};
template <> struct Num<float> : FloatNum<float> {
  static __device__ __forceinline__ bool divides(float, float b) { return b != 0.0f; }
  static __device__ __forceinline__ float pow(float a, float b) { return powf(a, b); }
};
template <> struct Num<double> : FloatNum<double> {
  static __device__ __forceinline__ bool divides(double a, double b) {
    return !(fabs(a) * 2.2250738585072014e-308 >= fabs(b));
  }
  static __device__ __forceinline__ double pow(double a, double b) { return ::pow(a, b); }
};

template <typename I, typename U> struct IntNum {
  static constexpr bool isFloat = false;
  static __device__ __forceinline__ bool divides(I, I b) { return b != 0; }
  // NumPy's integer floor_divide and remainder (Python's conventions; the
  // most negative value divided by -1 wraps).  Zero divisors never reach a
  // store; they give 0 here.
  static __device__ __forceinline__ I floordiv(I a, I b) {
    if (b == 0)
      return 0;
    if (b == I(-1))
      return I(U(0) - U(a));
    I q = a / b;
    if (((a > 0) != (b > 0)) && q * b != a)
      --q;
    return q;
  }
  static __device__ __forceinline__ I mod(I a, I b) {
    if (b == 0 || b == I(-1))
      return 0;
    I r = a % b;
    if (r != 0 && ((r < 0) != (b < 0)))
      r += b;
    return r;
  }
  // Non-negative exponents only (the host refuses others); wraps like NumPy.
  static __device__ __forceinline__ I pow(I a, I b) {
    U result = 1, base = U(a);
    for (U e = U(b < 0 ? 0 : b); e != 0; e >>= 1) {
      if (e & 1)
        result *= base;
      base *= base;
    }
    return I(result);
  }
  static __device__ __forceinline__ bool finite(I) { return true; }
  static __device__ __forceinline__ I bitAnd(I a, I b) { return a & b; }
  static __device__ __forceinline__ I bitOr(I a, I b) { return a | b; }
  static __device__ __forceinline__ I bitXor(I a, I b) { return a ^ b; }
  // Shift counts outside the type's width give 0 or the sign, as NumPy does.
  static __device__ __forceinline__ I shl(I a, I b) {
    return U(b) < U(8 * sizeof(I)) ? I(U(a) << U(b)) : I(0);
  }
  static __device__ __forceinline__ I shr(I a, I b) {
    return U(b) < U(8 * sizeof(I)) ? I(a >> b) : I(a < 0 ? -1 : 0);
  }
  static __device__ __forceinline__ I inv(I a) { return ~a; }
  static __device__ __forceinline__ I absOf(I a) { return a < 0 ? I(U(0) - U(a)) : a; }
  // Not defined on integer tiles; the host refuses such programs.
  static __device__ __forceinline__ I div(I a, I) { return a; }
  static __device__ __forceinline__ I sqrtOf(I a) { return a; }
  static __device__ __forceinline__ I exp(I a) { return a; }
  static __device__ __forceinline__ I log(I a) { return a; }
};
template <> struct Num<int32_t> : IntNum<int32_t, uint32_t> {};
template <> struct Num<int64_t> : IntNum<int64_t, uint64_t> {};

// Wrapping sum, difference and product (signed overflow is undefined in C++,
// NumPy wraps).
template <typename T> __device__ __forceinline__ T addOf(T a, T b) {
  if constexpr (Num<T>::isFloat) return a + b;
  else { using U = typename std::make_unsigned<T>::type; return T(U(a) + U(b)); }
}
template <typename T> __device__ __forceinline__ T subOf(T a, T b) {
  if constexpr (Num<T>::isFloat) return a - b;
  else { using U = typename std::make_unsigned<T>::type; return T(U(a) - U(b)); }
}
template <typename T> __device__ __forceinline__ T mulOf(T a, T b) {
  if constexpr (Num<T>::isFloat) return a * b;
  else { using U = typename std::make_unsigned<T>::type; return T(U(a) * U(b)); }
}
template <typename T> __device__ __forceinline__ T negOf(T a) {
  if constexpr (Num<T>::isFloat) return -a;
  else { using U = typename std::make_unsigned<T>::type; return T(U(0) - U(a)); }
}

template <typename T, int V> struct Packet { T v[V]; };

template <typename T, int V>
__device__ __forceinline__ Packet<T, V> loadPacket(const T *p) {
  Packet<T, V> out;
  if constexpr (V * sizeof(T) == 16) {
    const float4 raw = __ldcs(reinterpret_cast<const float4 *>(p));
    *reinterpret_cast<float4 *>(out.v) = raw;
  } else {
    out.v[0] = __ldcs(p);
  }
  return out;
}

template <typename T, int V>
__device__ __forceinline__ void storePacket(T *p, const Packet<T, V> &value) {
  if constexpr (V * sizeof(T) == 16)
    __stcs(reinterpret_cast<float4 *>(p), *reinterpret_cast<const float4 *>(value.v));
  else
    __stcs(p, value.v[0]);
}

// A load that leaves the line in the caches (a later pass of a row program
// reads the row again), where loadPacket streams.
template <typename T, int V>
__device__ __forceinline__ Packet<T, V> loadPacketKept(const T *p) {
  Packet<T, V> out;
  if constexpr (V * sizeof(T) == 16)
    *reinterpret_cast<float4 *>(out.v) = *reinterpret_cast<const float4 *>(p);
  else
    out.v[0] = *p;
  return out;
}

template <typename T> __device__ __forceinline__ T lowest();
template <> __device__ __forceinline__ float lowest<float>() { return -INFINITY; }
template <> __device__ __forceinline__ double lowest<double>() { return -INFINITY; }

// The larger of two values, NaN if either is NaN (what NumPy's max along an
// axis gives); one instruction for float.
__device__ __forceinline__ float maxNan(float a, float b) {
  float out;
  asm("max.NaN.f32 %0, %1, %2;" : "=f"(out) : "f"(a), "f"(b));
  return out;
}
__device__ __forceinline__ double maxNan(double a, double b) { return maxOf(a, b); }

// Floor division, remainder and power, one element at a time and out of line:
// their code is long (fmod, pow) and they are rare, so they must not cost the
// common operations registers.  `op` is one of the six (forward and reversed);
// returns the result and clears `valid` where numpy.ma would mask it.
template <typename T>
__device__ __noinline__ T rareBinary(uint32_t op, T a, T b, bool &valid) {
  using N = Num<T>;
  switch (op) {
  case HC_MAP_FLOORDIV: valid = N::divides(a, b); return N::floordiv(a, b);
  case HC_MAP_RFLOORDIV: valid = N::divides(b, a); return N::floordiv(b, a);
  case HC_MAP_MOD: valid = N::divides(a, b); return N::mod(a, b);
  case HC_MAP_RMOD: valid = N::divides(b, a); return N::mod(b, a);
  case HC_MAP_POW: {
    const T r = N::pow(a, b);
    valid = N::finite(r);
    return r;
  }
  default: {
    const T r = N::pow(b, a);
    valid = N::finite(r);
    return r;
  }
  }
}

// The binary operations of the machine on W accumulators; `operand(i)` names
// the second operand of element i (a register, a uniform value or an
// expression of the element's position), so that no operand is copied before
// it is used.  `ok` holds one validity bit per element; the division-like
// operations clear it where numpy.ma would mask the result.  EXTENDED: the
// whole operator table; otherwise (row programs) the nine operations up to
// `min` only, without validity.
template <typename T, int W, bool EXTENDED, typename F>
__device__ __forceinline__ void binary(uint32_t op, T (&acc)[W], F operand, uint32_t &ok) {
  using N = Num<T>;
#define HC_MAP_EACH(expr)                                                               \
  _Pragma("unroll") for (int i = 0; i < W; ++i) {                                       \
    const T a = acc[i], b = operand(i);                                                 \
    (void)a;                                                                            \
    acc[i] = (expr);                                                                    \
  }                                                                                     \
  break
  // `dividend` / `divisor` name a and b in the order the operation divides them.
#define HC_MAP_EACH_DIVIDING(dividend, divisor, expr)                                   \
  _Pragma("unroll") for (int i = 0; i < W; ++i) {                                       \
    const T a = acc[i], b = operand(i);                                                 \
    if (EXTENDED && !N::divides(dividend, divisor))                                     \
      ok &= ~(1u << i);                                                                 \
    acc[i] = (expr);                                                                    \
  }                                                                                     \
  break
  if (EXTENDED && op >= HC_MAP_FLOORDIV && op <= HC_MAP_RPOW) {
#pragma unroll
    for (int i = 0; i < W; ++i) {
      bool valid;
      acc[i] = rareBinary<T>(op, acc[i], operand(i), valid);
      if (!valid)
        ok &= ~(1u << i);
    }
    return;
  }
  switch (op) {
  case HC_MAP_LOAD: HC_MAP_EACH(b);
  case HC_MAP_ADD: HC_MAP_EACH(addOf(a, b));
  case HC_MAP_SUB: HC_MAP_EACH(subOf(a, b));
  case HC_MAP_RSUB: HC_MAP_EACH(subOf(b, a));
  case HC_MAP_MUL: HC_MAP_EACH(mulOf(a, b));
  case HC_MAP_DIV: HC_MAP_EACH_DIVIDING(a, b, N::div(a, b));
  case HC_MAP_RDIV: HC_MAP_EACH_DIVIDING(b, a, N::div(b, a));
  case HC_MAP_MAX: HC_MAP_EACH(maxOf(a, b));
  case HC_MAP_MIN: HC_MAP_EACH(minOf(a, b));
  default: break;
  }
  if (!EXTENDED)
    return;
  switch (op) {
  case HC_MAP_LT: HC_MAP_EACH(T(a < b));
  case HC_MAP_LE: HC_MAP_EACH(T(a <= b));
  case HC_MAP_EQ: HC_MAP_EACH(T(a == b));
  case HC_MAP_NE: HC_MAP_EACH(T(a != b));
  case HC_MAP_GE: HC_MAP_EACH(T(a >= b));
  case HC_MAP_GT: HC_MAP_EACH(T(a > b));
  case HC_MAP_AND: HC_MAP_EACH(N::bitAnd(a, b));
  case HC_MAP_OR: HC_MAP_EACH(N::bitOr(a, b));
  case HC_MAP_XOR: HC_MAP_EACH(N::bitXor(a, b));
  case HC_MAP_SHL: HC_MAP_EACH(N::shl(a, b));
  case HC_MAP_SHR: HC_MAP_EACH(N::shr(a, b));
  case HC_MAP_RSHL: HC_MAP_EACH(N::shl(b, a));
  case HC_MAP_RSHR: HC_MAP_EACH(N::shr(b, a));
  default: break;
  }
#undef HC_MAP_EACH
#undef HC_MAP_EACH_DIVIDING
}

// Stores the UNROLL packets of a thread (packet u at `base + u * STRIDE` of the
// row) that lie inside the row.  A packet whose elements are all valid goes out
// as one streaming store; otherwise only its valid elements are written.
template <typename T, int V, int UNROLL, int STRIDE>
__device__ __forceinline__ void storeValid(T *rowOut, const T (&value)[V * UNROLL], uint32_t ok,
                                           long long base, long long perRow, bool whole) {
  constexpr uint32_t full = V >= 32 ? ~0u : (1u << V) - 1u;
#pragma unroll
  for (int u = 0; u < UNROLL; ++u) {
    const long long i = base + (long long)u * STRIDE;
    if (whole || i < perRow) {
      const uint32_t bits = (ok >> (u * V)) & full;
      if (bits == full) {
        Packet<T, V> packet;
#pragma unroll
        for (int e = 0; e < V; ++e)
          packet.v[e] = value[u * V + e];
        storePacket<T, V>(rowOut + i * V, packet);
      } else {
#pragma unroll
        for (int e = 0; e < V; ++e)
          if (bits & (1u << e))
            rowOut[i * V + e] = value[u * V + e];
      }
    }
  }
}

// Runs instructions [pcBegin, pcEnd) of the program on W elements.  The
// inputs and the accumulator live in registers; the temporaries, which few
// expressions need, in this thread's column of a shared-memory array, so that
// registers stay free for loads in flight.  The first instruction of a range
// is always a load of the accumulator (the host refuses other programs), so
// `acc` needs no initial value.
//
// INDEXED: `row` and `packet` say where the elements sit (element i is in
// packet `packet + (i / V) * STRIDE`, at position i % V of it) - programs
// written at work-item level use the indices themselves as operands.
// ROWS: `scalars` are the values earlier passes of a row program reduced.
// EXTENDED: the whole operator table with validity tracking - `ok` receives
// the validity bits of the result (all set on entry), `parkedOk` holds those of
// the three parked values, W <= 16 bits each.  Without it (row programs, and
// element-wise programs that neither divide nor use the later operators) the
// machine is the basic one and both stay untouched.
template <typename T, int W, int V, int NIN, bool INDEXED, bool ROWS, int STRIDE,
          int COLUMNS = THREADS, bool EXTENDED = false>
__device__ __forceinline__ void evaluate(const HcMapProgramDev &p, int pcBegin, int pcEnd,
                                         const T (&x)[NIN][W], T (&acc)[W],
                                         T (&temps)[3][W][COLUMNS], long long row,
                                         long long packet, const T (&scalars)[4], uint32_t &ok,
                                         uint64_t &parkedOk) {
  static_assert(!EXTENDED || W <= 16, "the parked validity bits are packed 16 per temporary");
  static_assert(!(ROWS && EXTENDED), "row programs take the basic operations only");
  using N = Num<T>;
  const int lane = threadIdx.x;
#define HC_MAP_EACH(expr)                                                               \
  _Pragma("unroll") for (int i = 0; i < W; ++i) {                                       \
    const T a = acc[i];                                                                 \
    acc[i] = (expr);                                                                    \
  }                                                                                     \
  break
  for (int pc = pcBegin; pc < pcEnd; ++pc) {
    const uint32_t ins = p.code[pc], op = ins & 0xffu, src = ins >> 8;
    if (EXTENDED ? hcMapIsBinary(op) : op <= HC_MAP_MIN) {
      if (EXTENDED && op == HC_MAP_LOAD)
        ok = ~0u; // a fresh value (a parked one brings its own bits, below)
      if (src >= HC_MAP_SRC_CONST) {
        // One value for all elements: a constant, a row scalar, the row index.
        if (INDEXED && src == HC_MAP_SRC_COL) {
          binary<T, W, EXTENDED>(op, acc, [&](int i) {
            return T((packet + (long long)(i / V) * STRIDE) * V + i % V);
          }, ok);
          continue;
        }
        T one;
        if (ROWS && src >= HC_MAP_SRC_SCALAR) {
          const uint32_t k = src - HC_MAP_SRC_SCALAR;
          one = k == 0 ? scalars[0] : k == 1 ? scalars[1] : k == 2 ? scalars[2] : scalars[3];
        } else if (INDEXED && src == HC_MAP_SRC_ROW) {
          one = T(row);
        } else {
          one = T(p.consts[src - HC_MAP_SRC_CONST]);
        }
        binary<T, W, EXTENDED>(op, acc, [&](int) { return one; }, ok);
      } else if (src >= HC_MAP_SRC_TEMP) {
        T v[W]; // shared memory may be indexed by the operand number, registers not
#pragma unroll
        for (int i = 0; i < W; ++i)
          v[i] = temps[src - HC_MAP_SRC_TEMP][i][lane];
        if (EXTENDED) { // a load takes the parked validity, any other operation joins it
          const uint32_t bits =
              uint32_t(parkedOk >> (16 * (src - HC_MAP_SRC_TEMP))) | 0xffff0000u;
          ok = op == HC_MAP_LOAD ? bits : ok & bits;
        }
        binary<T, W, EXTENDED>(op, acc, [&](int i) { return v[i]; }, ok);
      } else {
        // Named registers only: an indexed access would go to local memory.
        switch (src) {
        case 0: binary<T, W, EXTENDED>(op, acc, [&](int i) { return x[0][i]; }, ok); break;
        case 1: if constexpr (NIN > 1) binary<T, W, EXTENDED>(op, acc, [&](int i) { return x[1][i]; }, ok); break;
        case 2: if constexpr (NIN > 2) binary<T, W, EXTENDED>(op, acc, [&](int i) { return x[2][i]; }, ok); break;
        default: if constexpr (NIN > 3) binary<T, W, EXTENDED>(op, acc, [&](int i) { return x[3][i]; }, ok); break;
        }
      }
      continue;
    }
    switch (op) {
    case HC_MAP_NEG: HC_MAP_EACH(negOf(a));
    case HC_MAP_ABS: HC_MAP_EACH(N::absOf(a));
    case HC_MAP_EXP: HC_MAP_EACH(N::exp(a));
    case HC_MAP_SQRT: HC_MAP_EACH(N::sqrtOf(a));
    case HC_MAP_LOG: HC_MAP_EACH(N::log(a));
    case HC_MAP_INV:
      if (!EXTENDED)
        break;
      HC_MAP_EACH(N::inv(a));
    case HC_MAP_SAVE0:
    case HC_MAP_SAVE1:
    case HC_MAP_SAVE2: // park the accumulator
#pragma unroll
      for (int i = 0; i < W; ++i)
        temps[op - HC_MAP_SAVE0][i][lane] = acc[i];
      if (EXTENDED) {
        const int shift = 16 * (op - HC_MAP_SAVE0);
        parkedOk = (parkedOk & ~(0xffffull << shift)) | (uint64_t(ok & 0xffffu) << shift);
      }
      break;
    default: // the row reductions end a pass and are handled by the caller
      break;
    }
  }
#undef HC_MAP_EACH
}

} // namespace hcmap
