// Programs compiled ahead of time into straight-line kernels (row_fused.cu,
// map_fused.cu) and matched at run time by hcRowProgram / hcMapElements.
// Written by `python -m hc_b200.hckernel.precompiled` from the bodies listed in
// hc_b200/hckernel/precompiled.py: edit that list, not this file.
#pragma once

#include <stdint.h>

namespace hcfused {
struct row_centre {
  static constexpr int nin = 1, n = 7;
  static constexpr uint32_t code[7] = {0x0u, 0x11u, 0x1480u, 0x885u, 0x193u, 0x0u, 0x1502u};
};
struct row_l2_normalise {
  static constexpr int nin = 1, n = 8;
  static constexpr uint32_t code[8] = {0x0u, 0x4u, 0x11u, 0x1480u, 0x8cu, 0x193u, 0x0u, 0x1505u};
};
struct row_log_softmax {
  static constexpr int nin = 1, n = 12;
  static constexpr uint32_t code[12] = {0x0u, 0x12u, 0x0u, 0x1402u, 0xbu, 0x111u, 0x1580u, 0x90u, 0x293u, 0x0u, 0x1402u, 0x1602u};
};
struct row_softmax_temperature {
  static constexpr int nin = 1, n = 12;
  static constexpr uint32_t code[12] = {0x0u, 0x12u, 0x0u, 0x1402u, 0x804u, 0xbu, 0x111u, 0x0u, 0x1402u, 0x804u, 0xbu, 0x1505u};
};
struct row_scaled_difference {
  static constexpr int nin = 2, n = 9;
  static constexpr uint32_t code[9] = {0x0u, 0xau, 0x12u, 0x1480u, 0x887u, 0x193u, 0x0u, 0x102u, 0x1505u};
};
struct row_standardise {
  static constexpr int nin = 1, n = 20;
  static constexpr uint32_t code[20] = {0x0u, 0x11u, 0x1480u, 0x885u, 0x293u, 0x0u, 0x1602u, 0xdu, 0x0u, 0x1602u, 0x404u, 0x111u, 0x1580u, 0x885u, 0x981u, 0x8cu, 0x393u, 0x0u, 0x1602u, 0x1705u};
};
struct row_rms_normalise {
  static constexpr int nin = 1, n = 10;
  static constexpr uint32_t code[10] = {0x0u, 0x4u, 0x11u, 0x1480u, 0x985u, 0x881u, 0x8cu, 0x193u, 0x0u, 0x1505u};
};
struct row_max_normalise {
  static constexpr int nin = 1, n = 5;
  static constexpr uint32_t code[5] = {0x0u, 0xau, 0x12u, 0x0u, 0x1405u};
};
struct row_sum_normalise {
  static constexpr int nin = 1, n = 4;
  static constexpr uint32_t code[4] = {0x0u, 0x11u, 0x0u, 0x1405u};
};
struct map_relu_axpby {
  static constexpr int nin = 2, n = 4;
  static constexpr uint32_t code[4] = {0x100u, 0x904u, 0x2u, 0x807u};
};
struct map_axpby {
  static constexpr int nin = 2, n = 6;
  static constexpr uint32_t code[6] = {0x0u, 0x804u, 0xdu, 0x100u, 0x904u, 0x401u};
};
struct map_axpy {
  static constexpr int nin = 2, n = 3;
  static constexpr uint32_t code[3] = {0x100u, 0x804u, 0x1u};
};
struct map_scale_shift {
  static constexpr int nin = 1, n = 3;
  static constexpr uint32_t code[3] = {0x0u, 0x904u, 0x801u};
};
struct map_scale {
  static constexpr int nin = 1, n = 2;
  static constexpr uint32_t code[2] = {0x0u, 0x804u};
};
struct map_relu {
  static constexpr int nin = 1, n = 2;
  static constexpr uint32_t code[2] = {0x0u, 0x807u};
};
struct map_clamp {
  static constexpr int nin = 1, n = 3;
  static constexpr uint32_t code[3] = {0x0u, 0x907u, 0x808u};
};
struct map_square_plus {
  static constexpr int nin = 1, n = 3;
  static constexpr uint32_t code[3] = {0x0u, 0x4u, 0x801u};
};
struct map_gauss {
  static constexpr int nin = 1, n = 4;
  static constexpr uint32_t code[4] = {0x0u, 0x4u, 0x9u, 0xbu};
};
struct map_poly4 {
  static constexpr int nin = 1, n = 9;
  static constexpr uint32_t code[9] = {0x0u, 0xc04u, 0xb01u, 0x4u, 0xa01u, 0x4u, 0x902u, 0x4u, 0x801u};
};
struct map_add {
  static constexpr int nin = 2, n = 2;
  static constexpr uint32_t code[2] = {0x100u, 0x1u};
};
struct map_sub {
  static constexpr int nin = 2, n = 2;
  static constexpr uint32_t code[2] = {0x100u, 0x2u};
};
struct map_mul {
  static constexpr int nin = 2, n = 2;
  static constexpr uint32_t code[2] = {0x100u, 0x4u};
};
struct map_div {
  static constexpr int nin = 2, n = 2;
  static constexpr uint32_t code[2] = {0x100u, 0x5u};
};
struct map_abs_difference {
  static constexpr int nin = 2, n = 3;
  static constexpr uint32_t code[3] = {0x100u, 0x2u, 0xau};
};
struct map_squared_difference {
  static constexpr int nin = 2, n = 6;
  static constexpr uint32_t code[6] = {0x100u, 0x2u, 0xdu, 0x100u, 0x2u, 0x404u};
};
struct map_hypot {
  static constexpr int nin = 2, n = 7;
  static constexpr uint32_t code[7] = {0x0u, 0x4u, 0xdu, 0x100u, 0x104u, 0x401u, 0xcu};
};
struct map_mixed {
  static constexpr int nin = 2, n = 16;
  static constexpr uint32_t code[16] = {0x0u, 0x9u, 0xdu, 0x100u, 0x8u, 0x404u, 0xdu, 0x100u, 0xau, 0xcu, 0x801u, 0xeu, 0x100u, 0x1u, 0x505u, 0x402u};
};
struct map_three_inputs {
  static constexpr int nin = 3, n = 11;
  static constexpr uint32_t code[11] = {0x0u, 0x4u, 0x801u, 0xdu, 0x100u, 0x2u, 0xeu, 0x200u, 0x102u, 0x504u, 0x405u};
};
struct map_multiply_add {
  static constexpr int nin = 3, n = 3;
  static constexpr uint32_t code[3] = {0x200u, 0x104u, 0x1u};
};
} // namespace hcfused

#define HC_FUSED_ROW_LIST(X) \
  X(centre) \
  X(l2_normalise) \
  X(log_softmax) \
  X(softmax_temperature) \
  X(scaled_difference) \
  X(standardise) \
  X(rms_normalise) \
  X(max_normalise) \
  X(sum_normalise)

#define HC_FUSED_MAP_LIST(X) \
  X(relu_axpby) \
  X(axpby) \
  X(axpy) \
  X(scale_shift) \
  X(scale) \
  X(relu) \
  X(clamp) \
  X(square_plus) \
  X(gauss) \
  X(poly4) \
  X(add) \
  X(sub) \
  X(mul) \
  X(div) \
  X(abs_difference) \
  X(squared_difference) \
  X(hypot) \
  X(mixed) \
  X(three_inputs) \
  X(multiply_add)
