// Parameter block of the element-wise expression kernel (map_elements.cu),
// shared by the kernel and by the host code that fills it.
#pragma once

#include <stdint.h>

// The expression is a program for a one-accumulator machine with three
// temporaries.  An instruction is `op | (src << 8)`; binary operations combine
// the accumulator with the operand `src` names.
enum HcMapOp : uint32_t {
  HC_MAP_LOAD = 0,  // acc = v
  HC_MAP_ADD = 1,   // acc = acc + v
  HC_MAP_SUB = 2,   // acc = acc - v
  HC_MAP_RSUB = 3,  // acc = v - acc
  HC_MAP_MUL = 4,   // acc = acc * v
  HC_MAP_DIV = 5,   // acc = acc / v
  HC_MAP_RDIV = 6,  // acc = v / acc
  HC_MAP_MAX = 7,   // acc = max(acc, v), NaN if either is NaN
  HC_MAP_MIN = 8,   // acc = min(acc, v), NaN if either is NaN
  HC_MAP_NEG = 9,   // acc = -acc
  HC_MAP_ABS = 10,  // acc = |acc|
  HC_MAP_EXP = 11,  // acc = exp(acc)
  HC_MAP_SQRT = 12, // acc = sqrt(acc)
  HC_MAP_SAVE0 = 13, // t0 = acc
  HC_MAP_SAVE1 = 14, // t1 = acc
  HC_MAP_SAVE2 = 15, // t2 = acc
  HC_MAP_LOG = 16,   // acc = log(acc)
  // Row programs only (row_program.cu): end a pass over the row by reducing the
  // accumulator along it into row scalar s[src].
  HC_MAP_RSUM = 17,
  HC_MAP_RMAX = 18,
  // Row programs only, in the uniform prologue of a pass: s[src] = acc.
  HC_MAP_SET = 19,
  // The rest of the tile operator table (element-wise kernel only).  The
  // division-like operations mark the element invalid where NumPy's masked
  // arrays mask it - a zero divisor; a power that is not finite - and an
  // invalid element is not stored, like the reference's masked store.
  HC_MAP_FLOORDIV = 20,  // acc = floor(acc / v), NumPy's floor_divide
  HC_MAP_RFLOORDIV = 21, // acc = floor(v / acc)
  HC_MAP_MOD = 22,       // acc = acc mod v, sign of the divisor (NumPy's remainder)
  HC_MAP_RMOD = 23,      // acc = v mod acc
  HC_MAP_POW = 24,       // acc = acc ** v
  HC_MAP_RPOW = 25,      // acc = v ** acc
  HC_MAP_LT = 26,        // acc = acc < v ? 1 : 0, and likewise:
  HC_MAP_LE = 27,
  HC_MAP_EQ = 28,
  HC_MAP_NE = 29,
  HC_MAP_GE = 30,
  HC_MAP_GT = 31,
  HC_MAP_AND = 32,       // integers: bitwise; floats: logical on zero / nonzero
  HC_MAP_OR = 33,
  HC_MAP_XOR = 34,
  HC_MAP_SHL = 35,       // integers only: acc << v
  HC_MAP_SHR = 36,       // acc >> v (arithmetic)
  HC_MAP_RSHL = 37,      // v << acc
  HC_MAP_RSHR = 38,      // v >> acc
  HC_MAP_INV = 39,       // integers: ~acc; floats (truth values): acc == 0 ? 1 : 0
  HC_MAP_OP_COUNT = 40
};
// Does `op` combine the accumulator with an operand (as opposed to changing
// the accumulator alone, saving it or ending a pass)?
#ifdef __CUDACC__
__host__ __device__
#endif
constexpr bool hcMapIsBinary(uint32_t op) {
  return op <= HC_MAP_MIN || (op >= HC_MAP_FLOORDIV && op <= HC_MAP_RSHR);
}
// Row programs only: an instruction with this bit set in its operation byte is
// uniform - it works on one value per row (operands: constants and row
// scalars) and runs once, before the pass walks the row.  A pass may begin
// with such instructions; they end in HC_MAP_SET.
constexpr uint32_t HC_MAP_UNIFORM = 0x80;

// Operand names: inputs 0..3, temporaries t0..t2, constants 0..7, and the row
// and column index of the element itself (as a value of the element type).
constexpr uint32_t HC_MAP_SRC_INPUT = 0, HC_MAP_SRC_TEMP = 4, HC_MAP_SRC_CONST = 8;
constexpr uint32_t HC_MAP_SRC_ROW = 16, HC_MAP_SRC_COL = 17;
// Row programs only: the row scalars s0..s3 that earlier passes reduced.
constexpr uint32_t HC_MAP_SRC_SCALAR = 20;
constexpr int HC_MAP_MAX_SCALARS = 4;
constexpr int HC_MAP_MAX_INPUTS = 4, HC_MAP_MAX_CONSTS = 8, HC_MAP_MAX_INSTR = 32;

struct HcMapProgramDev {
  const void *in[HC_MAP_MAX_INPUTS];
  int64_t inPitch[HC_MAP_MAX_INPUTS]; // in elements
  void *out;
  int64_t outPitch;
  int64_t rows, cols;
  int32_t nInputs, nInstr;
  uint32_t code[HC_MAP_MAX_INSTR];
  double consts[HC_MAP_MAX_CONSTS];
};
