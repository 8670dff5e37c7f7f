// Arithmetic of the per-token (AQ_SCALE_TOKEN) activation quantizer, shared by the quantizer
// kernels (aq_quantize.cu) and the decode kernel that quantizes its own activations
// (aq_direct_decode.cu), so that both produce the same integers and scales by construction.
#pragma once

#include "aq_common.cuh"

namespace aq {

// scale of a row from its absolute maximum, and the reciprocal used for the fast path below
__device__ __forceinline__ float token_scale_of(float row_absmax) {
  return fmaxf(__fdiv_rn(row_absmax, 127.0f), 1.0e-12f);
}

// rint(v / scale) with IEEE division semantics at the cost of a multiply: v * (1/scale)
// differs from the correctly rounded quotient by less than 2^-22 * |quotient| < 4e-5 for
// |quotient| <= 128, so both round to the same integer unless the product lies within 1e-4
// of a rounding boundary; only then is the division evaluated.
__device__ __forceinline__ int quantize_token_value(float v, float scale, float inv_scale) {
  const float t = __fmul_rn(v, inv_scale);
  int r = __float2int_rn(t);
  if (fabsf(t - static_cast<float>(r)) > 0.5f - 1.0e-4f || fabsf(t) > 128.0f) r = __float2int_rn(__fdiv_rn(v, scale));
  return max(-127, min(127, r));
}

__device__ __forceinline__ uint32_t pack4(int a, int b, int c, int d) {
  return (static_cast<uint32_t>(a) & 0xffu) | ((static_cast<uint32_t>(b) & 0xffu) << 8) |
         ((static_cast<uint32_t>(c) & 0xffu) << 16) | ((static_cast<uint32_t>(d) & 0xffu) << 24);
}

// Eight fp16 or bf16 values (one 16-byte vector) as floats.
__device__ __forceinline__ void unpack8(const uint4& raw, bool bf16, float (&v)[8]) {
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    if (bf16) {
      v[2 * i] = __uint_as_float(w[i] << 16);
      v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    } else {
      const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
      v[2 * i] = f.x;
      v[2 * i + 1] = f.y;
    }
  }
}

}  // namespace aq
