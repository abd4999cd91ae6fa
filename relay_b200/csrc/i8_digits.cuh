// Activations as int8 digits for the integer tensor-core linear (umma_i8_gemm.cu): a row of fp16
// values becomes x = 2^(e-20) * (d0 + 128 d1 + 128^2 d2) with 2^e above the row's largest
// magnitude and signed base-128 digits. Shared by the kernels that write digits: the pass of
// its own, the GEMM that makes them in shared memory, and RMSNorm when it feeds such a GEMM.
#pragma once
#include <cuda_fp16.h>

#include <cstdint>

namespace rb200 {
namespace i8d {

constexpr int kDigits = 3;
constexpr int kFracBits = 20;  // |fixed-point activation| < 2^20 = 64 * 128^2

__device__ __forceinline__ float abs_max8(const uint4& v) {
  const __half2* h = reinterpret_cast<const __half2*>(&v);
  const __half2 m = __hmax2(__hmax2(__habs2(h[0]), __habs2(h[1])), __hmax2(__habs2(h[2]), __habs2(h[3])));
  return fmaxf(__low2float(m), __high2float(m));
}

// One value -> its digits, each added into byte `lane` of w[g].
__device__ __forceinline__ void add_digits(float v, float up, int lane, uint32_t (&w)[kDigits]) {
  int X = __float2int_rn(v * up);  // |X| < 2^20
#pragma unroll
  for (int g = 0; g < kDigits; ++g) {
    // signed digit in [-64, 63]; the last one takes what is left (|.| <= 64)
    const int d = g == kDigits - 1 ? X : ((X + 64) & 127) - 64;
    w[g] |= static_cast<uint32_t>(d & 0xff) << (8 * lane);
    X = (X - d) >> 7;
  }
}

// Eight halves -> eight bytes (two words) of each digit.
__device__ __forceinline__ void digits8(const uint4& v, float up, uint32_t (&w)[kDigits][2]) {
  const __half* h = reinterpret_cast<const __half*>(&v);
  uint32_t lo[kDigits] = {}, hi[kDigits] = {};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    add_digits(__half2float(h[i]), up, i, lo);
    add_digits(__half2float(h[4 + i]), up, i, hi);
  }
#pragma unroll
  for (int g = 0; g < kDigits; ++g) {
    w[g][0] = lo[g];
    w[g][1] = hi[g];
  }
}

// Four halves -> one word of each digit.
__device__ __forceinline__ void digits4(const uint2& v, float up, uint32_t (&w)[kDigits]) {
  const __half* h = reinterpret_cast<const __half*>(&v);
#pragma unroll
  for (int g = 0; g < kDigits; ++g) w[g] = 0u;
#pragma unroll
  for (int i = 0; i < 4; ++i) add_digits(__half2float(h[i]), up, i, w);
}

// The row's scale pair from its largest magnitude: 2^e > mx (frexp: mx = m 2^e with m in
// [0.5, 1)); exact powers of two; an all-zero row keeps scale 0.
__device__ __forceinline__ void digit_scales(float mx, float& up, float& down) {
  int e = 0;
  if (mx > 0.f) frexpf(mx, &e);
  up = mx > 0.f ? ldexpf(1.0f, kFracBits - e) : 0.f;
  down = mx > 0.f ? ldexpf(1.0f, e - kFracBits) : 0.f;
}

}  // namespace i8d
}  // namespace rb200
