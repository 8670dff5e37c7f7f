// Per-tile arithmetic shared by the two small-M kernels (aq_stream.cu, aq_decode.cu).
//
// A warp owns 8 output columns (n = 8*warp + g) of a 64x64 weight tile that sits in
// shared memory in the prepared-image layout, and up to 16 activation rows per MMA.
// Lane (g, c) = (lane / 4, lane % 4) reads ONE 16-byte vector of weights -- column n,
// k in [16c, 16c+16) -- and one 16-byte vector of activations per row (rows g, g+8,
// same k range); both loads are bank-conflict free by construction of the layouts.
// The four 32-bit words of a vector feed two mma.sync.m16n8k32.s8 instructions; the
// MMA's own contraction index is a permutation of k that is identical for both
// operands, so the sums are the exact integer dot products over the tile's 64 k.
#pragma once

#include "aq_common.cuh"

namespace aq {

__device__ __forceinline__ void mma_s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                       uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// d = a * b (a fresh integer sum: the accumulator input is the constant zero)
__device__ __forceinline__ void mma_s8_fresh(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                             uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
      : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}

// Weight vector of lane (g, c) for output column n of a staged tile.
//   W8 tile: row n is 64 bytes, 16-byte chunk c stored at slot c ^ ((n >> 1) & 3).
//   W4 tile: row n is 32 bytes, chunk h = c / 2 holds k in [32h, 32h+32): low nibbles
//            k in [32h, 32h+16), high nibbles k in [32h+16, 32h+32).  The nibble plane
//            of this lane is widened to bytes holding 16*w.
__device__ __forceinline__ uint4 load_weight_vector(const uint8_t* tile, bool is_w4, int n, int c) {
  if (is_w4) {
    uint4 p = *reinterpret_cast<const uint4*>(tile + n * 32 + (c >> 1) * 16);
    const int shift = (c & 1) ? 0 : 4;
    p.x = (p.x << shift) & 0xf0f0f0f0u;
    p.y = (p.y << shift) & 0xf0f0f0f0u;
    p.z = (p.z << shift) & 0xf0f0f0f0u;
    p.w = (p.w << shift) & 0xf0f0f0f0u;
    return p;
  }
  return *reinterpret_cast<const uint4*>(tile + n * 64 + ((c ^ ((n >> 1) & 3)) << 4));
}

// d[0..1]: row g, columns 2c, 2c+1 of the warp's 8; d[2..3]: row g + 8.
__device__ __forceinline__ void tile_dot(int (&d)[4], const uint4& x_lo, const uint4& x_hi, const uint4& w) {
  d[0] = d[1] = d[2] = d[3] = 0;
  mma_s8(d, x_lo.x, x_hi.x, x_lo.y, x_hi.y, w.x, w.y);
  mma_s8(d, x_lo.z, x_hi.z, x_lo.w, x_hi.w, w.z, w.w);
}

// acc += float(d) * scale with separately rounded multiply and add.
__device__ __forceinline__ void tile_accumulate(float (&acc)[4], const int (&d)[4], float s_lo, float s_hi) {
  acc[0] = __fadd_rn(acc[0], __fmul_rn(static_cast<float>(d[0]), s_lo));
  acc[1] = __fadd_rn(acc[1], __fmul_rn(static_cast<float>(d[1]), s_lo));
  acc[2] = __fadd_rn(acc[2], __fmul_rn(static_cast<float>(d[2]), s_hi));
  acc[3] = __fadd_rn(acc[3], __fmul_rn(static_cast<float>(d[3]), s_hi));
}

// ---- helpers of the warp-per-tile kernels ------------------------------------------
// There the weights are the 16-row MMA operand (16 output columns per MMA pair) and up
// to eight activation rows ("tokens") the 8-column operand.

__device__ __forceinline__ uint4 ldg_x(const int8_t* p) {
  uint4 v;
  asm volatile("ld.global.nc.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

// payload bytes of tiles [first, last] given their records (tiles are contiguous)
__device__ __forceinline__ uint32_t span_bytes(const TileRecord& first, const TileRecord& last) {
  const uint32_t units = (last.offset_flag & ~kW4Flag) + ((last.offset_flag & kW4Flag) ? 1u : 2u) -
                         (first.offset_flag & ~kW4Flag);
  return units * kW4TileBytes;
}

// 16-byte weight vector at a precomputed lane offset of a staged tile; W4 nibbles are
// widened to bytes holding 16*w.
__device__ __forceinline__ uint4 weight_vector(const uint8_t* tile, bool is_w4, uint32_t w8_off, uint32_t w4_off,
                                               int w4_shift) {
  uint4 v = *reinterpret_cast<const uint4*>(tile + (is_w4 ? w4_off : w8_off));
  if (is_w4) {
    v.x = (v.x << w4_shift) & 0xf0f0f0f0u;
    v.y = (v.y << w4_shift) & 0xf0f0f0f0u;
    v.z = (v.z << w4_shift) & 0xf0f0f0f0u;
    v.w = (v.w << w4_shift) & 0xf0f0f0f0u;
  }
  return v;
}

__device__ __forceinline__ void store_any(void* out, int dtype, int64_t index, float value) {
  if (dtype == AQ_F32) {
    static_cast<float*>(out)[index] = value;
  } else if (dtype == AQ_BF16) {
    static_cast<__nv_bfloat16*>(out)[index] = __float2bfloat16_rn(value);
  } else {
    static_cast<__half*>(out)[index] = __float2half_rn(value);
  }
}

}  // namespace aq
