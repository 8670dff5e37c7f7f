// Activation quantizer kernels: fp16/bf16/fp32 rows -> int8 plus float32 scales.
//
// Two contracts (see include/alignquant_b200.h):
//   AQ_SCALE_TILE  one scale per 16-row x 64-column tile, endpoint rule and FP64
//                  rounding of the reference kernel
//                  (alignquant/kernels/cuda/linear.cu:453-603), optional structured
//                  64-point transform of every 64-column block first;
//   AQ_SCALE_TOKEN one scale per row, IEEE float32 arithmetic; also fused with the RMSNorm
//                  that precedes a decoder's qkv and gate/up projections.
// All are bandwidth-bound: 128-bit loads and stores, warp-shuffle reductions.
#include "aq_common.cuh"
#include "aq_ptx.cuh"
#include "aq_quantize_math.cuh"

namespace aq {
namespace {

template <typename T>
__device__ __forceinline__ void load16(const T* p, float (&v)[16]);

template <>
__device__ __forceinline__ void load16<__half>(const __half* p, float (&v)[16]) {
  const uint4 a = __ldg(reinterpret_cast<const uint4*>(p));
  const uint4 b = __ldg(reinterpret_cast<const uint4*>(p) + 1);
  const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const __half2 h = *reinterpret_cast<const __half2*>(&w[i]);
    const float2 f = __half22float2(h);
    v[2 * i] = f.x;
    v[2 * i + 1] = f.y;
  }
}

template <>
__device__ __forceinline__ void load16<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[16]) {
  const uint4 a = __ldg(reinterpret_cast<const uint4*>(p));
  const uint4 b = __ldg(reinterpret_cast<const uint4*>(p) + 1);
  const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    v[2 * i] = __uint_as_float(w[i] << 16);
    v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}

template <>
__device__ __forceinline__ void load16<float>(const float* p, float (&v)[16]) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float4 f = __ldg(reinterpret_cast<const float4*>(p) + i);
    v[4 * i] = f.x;
    v[4 * i + 1] = f.y;
    v[4 * i + 2] = f.z;
    v[4 * i + 3] = f.w;
  }
}

// ---------------------------------------------------------------------------
// AQ_SCALE_TOKEN: one CTA walks rows; pass 1 finds the row absmax, pass 2 divides and
// rounds.  Rows of up to 8192 values stay in registers between the passes (two 16-value
// chunks per thread); longer rows are read again (they are still in L1/L2).
// ---------------------------------------------------------------------------

__device__ __forceinline__ uint4 quantize_chunk(const float (&v)[16], float scale, float inv_scale) {
  int r[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) r[i] = quantize_token_value(v[i], scale, inv_scale);
  uint4 o;
  o.x = pack4(r[0], r[1], r[2], r[3]);
  o.y = pack4(r[4], r[5], r[6], r[7]);
  o.z = pack4(r[8], r[9], r[10], r[11]);
  o.w = pack4(r[12], r[13], r[14], r[15]);
  return o;
}

// Sixteen values as they come from memory (two 16-byte vectors of 16-bit values, four of floats):
// a row that waits in registers for its turn costs half the registers this way.
template <typename T>
struct Raw16 {
  uint4 part[sizeof(T) == 2 ? 2 : 4];
};

template <typename T>
__device__ __forceinline__ Raw16<T> load_raw16(const T* p) {
  Raw16<T> r;
#pragma unroll
  for (int i = 0; i < static_cast<int>(sizeof(r.part) / sizeof(uint4)); ++i) r.part[i] = __ldg(reinterpret_cast<const uint4*>(p) + i);
  return r;
}

__device__ __forceinline__ void raw_to_float(const Raw16<__half>& r, float (&v)[16]) {
  const uint32_t w[8] = {r.part[0].x, r.part[0].y, r.part[0].z, r.part[0].w, r.part[1].x, r.part[1].y, r.part[1].z, r.part[1].w};
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
    v[2 * i] = f.x;
    v[2 * i + 1] = f.y;
  }
}
__device__ __forceinline__ void raw_to_float(const Raw16<__nv_bfloat16>& r, float (&v)[16]) {
  const uint32_t w[8] = {r.part[0].x, r.part[0].y, r.part[0].z, r.part[0].w, r.part[1].x, r.part[1].y, r.part[1].z, r.part[1].w};
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    v[2 * i] = __uint_as_float(w[i] << 16);
    v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}
__device__ __forceinline__ void raw_to_float(const Raw16<float>& r, float (&v)[16]) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    v[4 * i] = __uint_as_float(r.part[i].x);
    v[4 * i + 1] = __uint_as_float(r.part[i].y);
    v[4 * i + 2] = __uint_as_float(r.part[i].z);
    v[4 * i + 3] = __uint_as_float(r.part[i].w);
  }
}

// Rows of up to 8192 values are read ONCE and wait in registers, as loaded, between the maximum
// and the rounding; the row a CTA takes next is requested before the current one is reduced, so
// that a CTA always has a row on its way from HBM (a CTA walks rows blockIdx.x, + gridDim.x, ...).
template <typename T>
__global__ void __launch_bounds__(256) quantize_token_kernel(const T* __restrict__ x,
                                                             int8_t* __restrict__ q,
                                                             float* __restrict__ scales,
                                                             int64_t m, int k) {
  __shared__ float warp_max[8];
  grid_launch_dependents();  // the consumer of q may start fetching its weights now
  grid_dependency_wait();    // x comes from the preceding kernel
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int chunks = k / 16;
  const bool in_registers = chunks <= 512;
  const int c0 = threadIdx.x, c1 = threadIdx.x + 256;
  Raw16<T> next0, next1;
  if (in_registers && blockIdx.x < m) {
    const T* first = x + static_cast<int64_t>(blockIdx.x) * k;
    if (c0 < chunks) next0 = load_raw16(first + c0 * 16);
    if (c1 < chunks) next1 = load_raw16(first + c1 * 16);
  }
  for (int64_t row = blockIdx.x; row < m; row += gridDim.x) {
    const T* xr = x + row * k;
    float amax = 0.0f;
    Raw16<T> r0, r1;
    if (in_registers) {
      r0 = next0;
      r1 = next1;
      const int64_t following = row + gridDim.x;
      if (following < m) {
        const T* xn = x + following * k;
        if (c0 < chunks) next0 = load_raw16(xn + c0 * 16);
        if (c1 < chunks) next1 = load_raw16(xn + c1 * 16);
      }
      float v[16];
      if (c0 < chunks) {
        raw_to_float(r0, v);
#pragma unroll
        for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(v[i]));
      }
      if (c1 < chunks) {
        raw_to_float(r1, v);
#pragma unroll
        for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(v[i]));
      }
    } else {
      for (int c = threadIdx.x; c < chunks; c += 256) {
        float v[16];
        load16(xr + c * 16, v);
#pragma unroll
        for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(v[i]));
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    if (lane == 0) warp_max[warp] = amax;
    __syncthreads();
    float block_max = warp_max[0];
#pragma unroll
    for (int w = 1; w < 8; ++w) block_max = fmaxf(block_max, warp_max[w]);
    const float scale = token_scale_of(block_max);
    const float inv_scale = __fdiv_rn(1.0f, scale);
    if (threadIdx.x == 0) scales[row] = scale;
    int8_t* qr = q + row * k;
    if (in_registers) {
      float v[16];
      if (c0 < chunks) {
        raw_to_float(r0, v);
        *reinterpret_cast<uint4*>(qr + c0 * 16) = quantize_chunk(v, scale, inv_scale);
      }
      if (c1 < chunks) {
        raw_to_float(r1, v);
        *reinterpret_cast<uint4*>(qr + c1 * 16) = quantize_chunk(v, scale, inv_scale);
      }
    } else {
      for (int c = threadIdx.x; c < chunks; c += 256) {
        float v[16];
        load16(xr + c * 16, v);
        *reinterpret_cast<uint4*>(qr + c * 16) = quantize_chunk(v, scale, inv_scale);
      }
    }
    __syncthreads();
  }
}

// ---------------------------------------------------------------------------
// RMSNorm + AQ_SCALE_TOKEN quantizer in one pass over the row.
//   r    = float(1 / sqrt(sum(x^2) / K + eps))      sum, division and root in FP64
//   n    = round_T(x * r)                            the normalised value in the activation type
//   y    = round_T(float(weight) * n)                what a decoder's RMSNorm module returns
//   s    = max(absmax(y) / 127, 1e-12),  q = rint(y / s) clamped to [-127, 127]
// (the arithmetic of the Llama / Qwen3 RMSNorm module followed by the per-token quantizer).
// One CTA per row; rows of up to 8192 values stay in registers between the three phases,
// longer rows are read again.
// ---------------------------------------------------------------------------

template <typename T>
__device__ __forceinline__ float round_to(float v);
template <>
__device__ __forceinline__ float round_to<__half>(float v) { return __half2float(__float2half_rn(v)); }
template <>
__device__ __forceinline__ float round_to<__nv_bfloat16>(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
template <>
__device__ __forceinline__ float round_to<float>(float v) { return v; }

template <typename T>
__device__ __forceinline__ void store16(T* p, const float (&v)[16]);
template <>
__device__ __forceinline__ void store16<__half>(__half* p, const float (&v)[16]) {
  uint32_t w[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const __half2 h = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
    w[i] = *reinterpret_cast<const uint32_t*>(&h);
  }
  reinterpret_cast<uint4*>(p)[0] = make_uint4(w[0], w[1], w[2], w[3]);
  reinterpret_cast<uint4*>(p)[1] = make_uint4(w[4], w[5], w[6], w[7]);
}
template <>
__device__ __forceinline__ void store16<__nv_bfloat16>(__nv_bfloat16* p, const float (&v)[16]) {
  uint32_t w[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    w[i] = *reinterpret_cast<const uint32_t*>(&h);
  }
  reinterpret_cast<uint4*>(p)[0] = make_uint4(w[0], w[1], w[2], w[3]);
  reinterpret_cast<uint4*>(p)[1] = make_uint4(w[4], w[5], w[6], w[7]);
}
template <>
__device__ __forceinline__ void store16<float>(float* p, const float (&v)[16]) {
#pragma unroll
  for (int i = 0; i < 4; ++i) reinterpret_cast<float4*>(p)[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
}

template <typename T>
__device__ __forceinline__ void normalise16(float (&v)[16], const T* weight, float r) {
  float w[16];
  load16(weight, w);
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = round_to<T>(__fmul_rn(w[i], round_to<T>(__fmul_rn(v[i], r))));
}

template <typename T>
__global__ void __launch_bounds__(256) rmsnorm_quantize_kernel(const T* __restrict__ x, const T* __restrict__ weight,
                                                               float eps, int8_t* __restrict__ q,
                                                               float* __restrict__ scales, T* __restrict__ normed,
                                                               int64_t m, int k) {
  __shared__ double warp_sum[8];
  __shared__ float warp_max[8];
  grid_launch_dependents();
  grid_dependency_wait();
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int chunks = k / 16;
  const bool in_registers = chunks <= 512;
  for (int64_t row = blockIdx.x; row < m; row += gridDim.x) {
    const T* xr = x + row * k;
    float v0[16], v1[16];
    const int c0 = threadIdx.x, c1 = threadIdx.x + 256;
    double ss = 0.0;
    if (in_registers) {
      if (c0 < chunks) {
        load16(xr + c0 * 16, v0);
#pragma unroll
        for (int i = 0; i < 16; ++i) ss += static_cast<double>(v0[i]) * static_cast<double>(v0[i]);
      }
      if (c1 < chunks) {
        load16(xr + c1 * 16, v1);
#pragma unroll
        for (int i = 0; i < 16; ++i) ss += static_cast<double>(v1[i]) * static_cast<double>(v1[i]);
      }
    } else {
      for (int c = threadIdx.x; c < chunks; c += 256) {
        float v[16];
        load16(xr + c * 16, v);
#pragma unroll
        for (int i = 0; i < 16; ++i) ss += static_cast<double>(v[i]) * static_cast<double>(v[i]);
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if (lane == 0) warp_sum[warp] = ss;
    __syncthreads();
    double total = warp_sum[0];
#pragma unroll
    for (int w = 1; w < 8; ++w) total += warp_sum[w];
    const float r = static_cast<float>(1.0 / sqrt(total / static_cast<double>(k) + static_cast<double>(eps)));

    float amax = 0.0f;
    if (in_registers) {
      if (c0 < chunks) {
        normalise16(v0, weight + c0 * 16, r);
#pragma unroll
        for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(v0[i]));
      }
      if (c1 < chunks) {
        normalise16(v1, weight + c1 * 16, r);
#pragma unroll
        for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(v1[i]));
      }
    } else {
      for (int c = threadIdx.x; c < chunks; c += 256) {
        float v[16];
        load16(xr + c * 16, v);
        normalise16(v, weight + c * 16, r);
#pragma unroll
        for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(v[i]));
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    if (lane == 0) warp_max[warp] = amax;
    __syncthreads();
    float block_max = warp_max[0];
#pragma unroll
    for (int w = 1; w < 8; ++w) block_max = fmaxf(block_max, warp_max[w]);
    const float scale = token_scale_of(block_max);
    const float inv_scale = __fdiv_rn(1.0f, scale);
    if (threadIdx.x == 0) scales[row] = scale;
    int8_t* qr = q + row * k;
    T* nr = normed != nullptr ? normed + row * k : nullptr;
    if (in_registers) {
      if (c0 < chunks) {
        *reinterpret_cast<uint4*>(qr + c0 * 16) = quantize_chunk(v0, scale, inv_scale);
        if (nr != nullptr) store16(nr + c0 * 16, v0);
      }
      if (c1 < chunks) {
        *reinterpret_cast<uint4*>(qr + c1 * 16) = quantize_chunk(v1, scale, inv_scale);
        if (nr != nullptr) store16(nr + c1 * 16, v1);
      }
    } else {
      for (int c = threadIdx.x; c < chunks; c += 256) {
        float v[16];
        load16(xr + c * 16, v);
        normalise16(v, weight + c * 16, r);
        *reinterpret_cast<uint4*>(qr + c * 16) = quantize_chunk(v, scale, inv_scale);
        if (nr != nullptr) store16(nr + c * 16, v);
      }
    }
    __syncthreads();
  }
}

// ---------------------------------------------------------------------------
// AQ_SCALE_TILE: one warp per (16-row group, 64-column block).
// ---------------------------------------------------------------------------

// rint(v / scale) with the reference's FP64 semantics.  v * (1/scale) differs from
// the correctly rounded quotient by < 1e-13 for |v/scale| <= 129, so it rounds to the
// same integer unless it lies within 1e-9 of a rounding boundary; only then is the
// exact division evaluated.
__device__ __forceinline__ int quantize_fp64(double v, double scale, double inv_scale) {
  const double t = v * inv_scale;
  int r = __double2int_rn(t);
  if (fabs(t - static_cast<double>(r)) > 0.5 - 1.0e-9) r = __double2int_rn(__ddiv_rn(v, scale));
  return max(-128, min(127, r));
}

template <typename T>
__global__ void __launch_bounds__(256) quantize_tile_kernel(const T* __restrict__ x,
                                                            const int32_t* __restrict__ v_metadata,
                                                            int8_t* __restrict__ q,
                                                            float* __restrict__ scales,
                                                            int64_t m, int n_k) {
  __shared__ float stage[8][kTile];
  grid_launch_dependents();
  grid_dependency_wait();
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int64_t m_tiles = (m + 15) / 16;
  const int64_t tile = static_cast<int64_t>(blockIdx.x) * 8 + warp;
  if (tile >= m_tiles * n_k) return;  // whole warps leave; only warp-level syncs below
  const int64_t mt = tile / n_k;
  const int kt = static_cast<int>(tile % n_k);
  const int64_t k = static_cast<int64_t>(n_k) * kTile;
  const int32_t* meta = v_metadata ? v_metadata + static_cast<int64_t>(kt) * 4 * kTile : nullptr;
  const bool identity = meta == nullptr || meta[0] == 0;

  if (identity) {
    // lane -> rows (lane/4, lane/4 + 8), 16 consecutive columns starting at 16*(lane%4)
    const int r0 = lane >> 2;
    const int c0 = (lane & 3) * 16;
    float v[2][16];
    float pos = 0.0f, neg = 0.0f;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int64_t row = mt * 16 + r0 + 8 * h;
      if (row < m) {
        load16(x + row * k + kt * kTile + c0, v[h]);
      } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) v[h][i] = 0.0f;
      }
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        pos = fmaxf(pos, v[h][i]);
        neg = fmaxf(neg, -v[h][i]);
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      pos = fmaxf(pos, __shfl_xor_sync(0xffffffffu, pos, o));
      neg = fmaxf(neg, __shfl_xor_sync(0xffffffffu, neg, o));
    }
    const double scale =
        fmax(fmax(static_cast<double>(pos) / 127.0, static_cast<double>(neg) / 128.0), 1.0e-12);
    const double inv_scale = 1.0 / scale;
    if (lane == 0) scales[mt * n_k + kt] = static_cast<float>(scale);
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int64_t row = mt * 16 + r0 + 8 * h;
      if (row < m) {
        int r[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) r[i] = quantize_fp64(static_cast<double>(v[h][i]), scale, inv_scale);
        uint4 o;
        o.x = pack4(r[0], r[1], r[2], r[3]);
        o.y = pack4(r[4], r[5], r[6], r[7]);
        o.z = pack4(r[8], r[9], r[10], r[11]);
        o.w = pack4(r[12], r[13], r[14], r[15]);
        *reinterpret_cast<uint4*>(q + row * k + kt * kTile + c0) = o;
      }
    }
    return;
  }

  // Structured transform V = diag(left) * H[perm, :] * diag(right) / 8 applied to each
  // row: scatter x[r]*left[r] to position perm[r], 64-point Walsh-Hadamard butterfly,
  // multiply by right and 1/8 -- all in FP64 like the reference.
  const int perm_lo = meta[kTile + lane];
  const int perm_hi = meta[kTile + lane + 32];
  const float left_lo = static_cast<float>(meta[2 * kTile + lane]);
  const float left_hi = static_cast<float>(meta[2 * kTile + lane + 32]);
  const double right_lo = static_cast<double>(meta[3 * kTile + lane]) * 0.125;
  const double right_hi = static_cast<double>(meta[3 * kTile + lane + 32]) * 0.125;
  double lo[16], hi[16];
  double pos = 0.0, neg = 0.0;
#pragma unroll
  for (int r = 0; r < 16; ++r) {
    const int64_t row = mt * 16 + r;
    float a = 0.0f, b = 0.0f;
    if (row < m) {
      a = to_float(x[row * k + kt * kTile + lane]);
      b = to_float(x[row * k + kt * kTile + lane + 32]);
    }
    __syncwarp();
    stage[warp][perm_lo] = a * left_lo;
    stage[warp][perm_hi] = b * left_hi;
    __syncwarp();
    double l = static_cast<double>(stage[warp][lane]);
    double h = static_cast<double>(stage[warp][lane + 32]);
    fwht64_warp(l, h, lane);
    lo[r] = l * right_lo;
    hi[r] = h * right_hi;
    pos = fmax(pos, fmax(lo[r], hi[r]));
    neg = fmax(neg, fmax(-lo[r], -hi[r]));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    pos = fmax(pos, __shfl_xor_sync(0xffffffffu, pos, o));
    neg = fmax(neg, __shfl_xor_sync(0xffffffffu, neg, o));
  }
  const double scale = fmax(fmax(pos / 127.0, neg / 128.0), 1.0e-12);
  const double inv_scale = 1.0 / scale;
  if (lane == 0) scales[mt * n_k + kt] = static_cast<float>(scale);
#pragma unroll
  for (int r = 0; r < 16; ++r) {
    const int64_t row = mt * 16 + r;
    if (row < m) {
      q[row * k + kt * kTile + lane] = static_cast<int8_t>(quantize_fp64(lo[r], scale, inv_scale));
      q[row * k + kt * kTile + lane + 32] = static_cast<int8_t>(quantize_fp64(hi[r], scale, inv_scale));
    }
  }
}

template <typename T>
int launch_typed(const void* x, int64_t m, int64_t k, const int32_t* v_metadata, int scale_mode,
                 int8_t* q, float* scales, cudaStream_t stream) {
  const T* xt = static_cast<const T*>(x);
  cudaLaunchConfig_t config = {};
  config.blockDim = dim3(256, 1, 1);
  config.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attr;
  config.numAttrs = use_dependent_launch() ? 1 : 0;
  cudaError_t status;
  if (scale_mode == AQ_SCALE_TOKEN) {
    const int64_t grid = m < 148 * 16 ? m : 148 * 16;
    config.gridDim = dim3(static_cast<unsigned>(grid), 1, 1);
    status = cudaLaunchKernelEx(&config, quantize_token_kernel<T>, xt, q, scales, m, static_cast<int>(k));
  } else {
    const int64_t tiles = (m + 15) / 16 * (k / kTile);
    config.gridDim = dim3(static_cast<unsigned>((tiles + 7) / 8), 1, 1);
    status = cudaLaunchKernelEx(&config, quantize_tile_kernel<T>, xt, v_metadata, q, scales, m,
                                static_cast<int>(k / kTile));
  }
  return check_cuda(status, "activation quantizer launch");
}

template <typename T>
int launch_rmsnorm_typed(const void* x, const void* weight, float eps, int64_t m, int64_t k, int8_t* q, float* scales,
                         void* normed, cudaStream_t stream) {
  cudaLaunchConfig_t config = {};
  config.blockDim = dim3(256, 1, 1);
  config.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attr;
  config.numAttrs = use_dependent_launch() ? 1 : 0;
  const int64_t grid = m < 148 * 16 ? m : 148 * 16;
  config.gridDim = dim3(static_cast<unsigned>(grid), 1, 1);
  return check_cuda(cudaLaunchKernelEx(&config, rmsnorm_quantize_kernel<T>, static_cast<const T*>(x),
                                       static_cast<const T*>(weight), eps, q, scales, static_cast<T*>(normed), m,
                                       static_cast<int>(k)),
                    "rmsnorm + quantizer launch");
}

}  // namespace

int launch_rmsnorm_quantize(const void* x, int x_dtype, int64_t m, int64_t k, const void* weight, float eps, int8_t* q,
                            float* scales, void* normed, cudaStream_t stream) {
  switch (x_dtype) {
    case AQ_F16:
      return launch_rmsnorm_typed<__half>(x, weight, eps, m, k, q, scales, normed, stream);
    case AQ_BF16:
      return launch_rmsnorm_typed<__nv_bfloat16>(x, weight, eps, m, k, q, scales, normed, stream);
    case AQ_F32:
      return launch_rmsnorm_typed<float>(x, weight, eps, m, k, q, scales, normed, stream);
    default:
      return fail(AQ_ERR_INVALID, "x_dtype must be AQ_F16, AQ_BF16 or AQ_F32, got %d", x_dtype);
  }
}

int launch_quantize(const void* x, int x_dtype, int64_t m, int64_t k, const int32_t* v_metadata,
                    int scale_mode, int8_t* q, float* scales, cudaStream_t stream) {
  switch (x_dtype) {
    case AQ_F16:
      return launch_typed<__half>(x, m, k, v_metadata, scale_mode, q, scales, stream);
    case AQ_BF16:
      return launch_typed<__nv_bfloat16>(x, m, k, v_metadata, scale_mode, q, scales, stream);
    case AQ_F32:
      return launch_typed<float>(x, m, k, v_metadata, scale_mode, q, scales, stream);
    default:
      return fail(AQ_ERR_INVALID, "x_dtype must be AQ_F16, AQ_BF16 or AQ_F32, got %d", x_dtype);
  }
}

}  // namespace aq
