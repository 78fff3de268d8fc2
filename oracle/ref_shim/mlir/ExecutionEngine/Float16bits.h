/* Stand-in for the upstream MLIR header of the same name (not part of the
 * reference tree).  TEST INFRASTRUCTURE ONLY, used to compile the reference's
 * CPU GEMM into oracle/_ref/.  Provides 16-bit storage types with a `bits`
 * member and a rounding (nearest-even) constructor from float. */
#ifndef IMEX_B200_SHIM_FLOAT16BITS_H
#define IMEX_B200_SHIM_FLOAT16BITS_H

#include <cstdint>
#include <iosfwd>

extern "C" {
uint16_t oracle_f32_to_bf16(float v);
uint16_t oracle_f32_to_f16(float v);
float oracle_bf16_to_f32(uint16_t bits);
float oracle_f16_to_f32(uint16_t bits);
}

struct f16 {
  f16() : bits(0) {}
  f16(float f) : bits(oracle_f32_to_f16(f)) {}
  uint16_t bits;
};

struct bf16 {
  bf16() : bits(0) {}
  bf16(float f) : bits(oracle_f32_to_bf16(f)) {}
  uint16_t bits;
};

#endif
