// Scalar stand-ins for src/kernels/cpu/vec.cpp and q8_0.cpp, which need <arm_neon.h>.
// Same contracts: elementwise conversion to F32 and dot products accumulated in F32.
#include <cstring>

#include "core/error.h"
#include "core/half.h"
#include "kernels/cpu/q8_0.h"
#include "kernels/cpu/vec.h"

namespace tie {

void to_f32(DType dtype, const void* src, float* dst, int64_t n) {
  if (dtype == DType::F32) {
    std::memcpy(dst, src, static_cast<size_t>(n) * sizeof(float));
  } else if (dtype == DType::F16) {
    for (int64_t i = 0; i < n; ++i) dst[i] = f16_to_f32(static_cast<const uint16_t*>(src)[i]);
  } else if (dtype == DType::BF16) {
    for (int64_t i = 0; i < n; ++i) dst[i] = bf16_to_f32(static_cast<const uint16_t*>(src)[i]);
  } else {
    fail<InvalidArgument>("to_f32: unsupported dtype in the scalar stand-in");
  }
}

float dot_f32(const float* x, const float* y, int64_t n) {
  float acc = 0.0f;
  for (int64_t i = 0; i < n; ++i) acc += x[i] * y[i];
  return acc;
}

float dot_f32_f16(const float* x, const uint16_t* w, int64_t n) {
  float acc = 0.0f;
  for (int64_t i = 0; i < n; ++i) acc += x[i] * f16_to_f32(w[i]);
  return acc;
}

float dot_f32_bf16(const float* x, const uint16_t* w, int64_t n) {
  float acc = 0.0f;
  for (int64_t i = 0; i < n; ++i) acc += x[i] * bf16_to_f32(w[i]);
  return acc;
}

void quantize_row_q8_0(const float*, BlockQ8_0*, int64_t) { fail<InvalidArgument>("Q8_0 is not part of this harness"); }
void dequantize_row_q8_0(const BlockQ8_0*, float*, int64_t) { fail<InvalidArgument>("Q8_0 is not part of this harness"); }
float dot_f32_q8_0(const float*, const BlockQ8_0*, int64_t) { fail<InvalidArgument>("Q8_0 is not part of this harness"); }

}  // namespace tie
