// C wrappers around the reference's own software number types, so that tests can call them
// through ctypes.  TEST INFRASTRUCTURE ONLY.  This file is compiled together with the
// reference's unmodified executor/lib/Runtime/Backend/Common/DataTypes.cpp (never copied into
// this repository) by oracle/Makefile; the result lands in oracle/_ref/.
#include "mlir-executor/Runtime/Backend/Common/DataTypes.h"
#include <cstdint>

using namespace mtrt;

extern "C" {
uint8_t ref_f32_to_f8e4m3(float v) { return static_cast<uint8_t>(F8E4M3FN(v).getRawBits()); }
float ref_f8e4m3_to_f32(uint8_t b) { return float(F8E4M3FN::fromRawBits(static_cast<int8_t>(b))); }
uint16_t ref_f32_to_f16(float v) { return static_cast<uint16_t>(Float16(v).getRawBits()); }
float ref_f16_to_f32(uint16_t b) { return float(Float16::fromRawBits(static_cast<int16_t>(b))); }
uint16_t ref_f32_to_bf16(float v) { return static_cast<uint16_t>(BFloat16(v).getRawBits()); }
float ref_bf16_to_f32(uint16_t b) { return float(BFloat16::fromRawBits(static_cast<int16_t>(b))); }
int ref_int4_saturate(int v) { return int(Int4(v)); }

void ref_f32_to_f8e4m3_n(const float *in, uint8_t *out, int64_t n) {
  for (int64_t i = 0; i < n; i++) out[i] = ref_f32_to_f8e4m3(in[i]);
}
void ref_f32_to_f16_n(const float *in, uint16_t *out, int64_t n) {
  for (int64_t i = 0; i < n; i++) out[i] = ref_f32_to_f16(in[i]);
}
void ref_f32_to_bf16_n(const float *in, uint16_t *out, int64_t n) {
  for (int64_t i = 0; i < n; i++) out[i] = ref_f32_to_bf16(in[i]);
}
}
