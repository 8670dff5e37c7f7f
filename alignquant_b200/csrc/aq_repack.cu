// One-time re-layout of a layer's artifact tensors into the prepared image.
//
// Source (alignquant/quantization/artifact.py:62-73, 131-199): per-precision arenas
// of 64x64 tiles in "Layout-B" physical order.  Element (k, n) of a tile is byte
//     256*(n/4) + 16*v + k%16,  v = 8*(k/32) + 4*(t/4) + ((t%4) ^ ((n/4)%4)),
//     t = (k/16)%2 + 2*(n%4),
// i.e. every aligned 16-byte vector holds 16 consecutive k of one output column.
// W4 tiles store the same order two values per byte, low nibble first.
//
// Destination (include/alignquant_b200.h): tiles in (j, k) order behind an array of
// 8-byte records.  A W8 tile is 64 rows (output columns n) of 64 bytes (k), the
// 16-byte chunk c = k/16 of row n stored at slot c ^ ((n/2) % 4): the K-major
// 64-byte-swizzle operand layout of tcgen05.mma, which also makes the small-M
// kernels' 16-byte shared-memory reads conflict free.  A W4 tile is 64 rows of 32
// bytes: chunk h = k/32 holds k%32 < 16 in the low nibbles and k%32 >= 16 in the high
// nibbles of the same bytes, so one shift-and-mask widens a word.
#include "aq_common.cuh"

namespace aq {
namespace {

__device__ __forceinline__ int layout_b_vector(int n, int k16) {
  const int vs = n >> 2;
  const int t = (k16 & 1) + 2 * (n & 3);
  const int v = 8 * (k16 >> 1) + 4 * (t >> 2) + ((t & 3) ^ (vs & 3));
  return vs * 16 + v;  // index of the 16-element vector inside the tile
}

__global__ void __launch_bounds__(256) repack_kernel(
    const uint8_t* __restrict__ state_bits, const uint8_t* __restrict__ w4_payload,
    const float* __restrict__ w4_scales, const int8_t* __restrict__ w8_payload,
    const float* __restrict__ w8_scales, const int32_t* __restrict__ w4_row_offsets,
    const int32_t* __restrict__ w8_row_offsets, int n_k, TileRecord* __restrict__ records,
    uint8_t* __restrict__ payload) {
  __shared__ int warp_count[8];
  const int64_t tile = blockIdx.x;
  const int j = static_cast<int>(tile / n_k);
  const int kt = static_cast<int>(tile % n_k);
  const int64_t row_base = static_cast<int64_t>(j) * n_k;

  // W4 tiles of row j that precede kt
  int count = 0;
  for (int i = threadIdx.x; i < kt; i += 256) {
    const int64_t bit = row_base + i;
    count += (state_bits[bit >> 3] >> (bit & 7)) & 1;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) count += __shfl_xor_sync(0xffffffffu, count, o);
  if ((threadIdx.x & 31) == 0) warp_count[threadIdx.x >> 5] = count;
  __syncthreads();
  int before4 = 0;
#pragma unroll
  for (int w = 0; w < 8; ++w) before4 += warp_count[w];
  const int before8 = kt - before4;
  const int64_t self_bit = row_base + kt;
  const bool is_w4 = ((state_bits[self_bit >> 3] >> (self_bit & 7)) & 1) != 0;
  const int64_t index4 = static_cast<int64_t>(w4_row_offsets[j]) + before4;
  const int64_t index8 = static_cast<int64_t>(w8_row_offsets[j]) + before8;
  const int64_t offset_units = index4 + 2 * index8;  // 2048-byte units
  uint8_t* dst = payload + offset_units * kW4TileBytes;

  if (threadIdx.x == 0) {
    TileRecord rec;
    rec.offset_flag = static_cast<uint32_t>(offset_units) | (is_w4 ? kW4Flag : 0u);
    rec.scale = is_w4 ? w4_scales[index4] * 0.0625f : w8_scales[index8];
    records[tile] = rec;
  }

  if (!is_w4) {
    // destination chunk r = 4*n + slot  <-  Layout-B vector of (n, k16 = slot ^ ((n/2)%4))
    const uint4* src = reinterpret_cast<const uint4*>(w8_payload + index8 * kW8TileBytes);
    const int r = threadIdx.x;
    const int n = r >> 2, slot = r & 3;
    reinterpret_cast<uint4*>(dst)[r] = src[layout_b_vector(n, slot ^ ((n >> 1) & 3))];
  } else if (threadIdx.x < 128) {
    // destination chunk u = 2*n + h; a source vector of 16 int4 is 8 bytes
    const uint2* src = reinterpret_cast<const uint2*>(w4_payload + index4 * kW4TileBytes);
    const int u = threadIdx.x;
    const int n = u >> 1, h = u & 1;
    const uint2 a = src[layout_b_vector(n, 2 * h)];      // k%32 in [0,16): nibble i = k offset i
    const uint2 b = src[layout_b_vector(n, 2 * h + 1)];  // k%32 in [16,32)
    const uint64_t av = (static_cast<uint64_t>(a.y) << 32) | a.x;
    const uint64_t bv = (static_cast<uint64_t>(b.y) << 32) | b.x;
    uint32_t out[4];
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      uint32_t word = 0;
#pragma unroll
      for (int byte = 0; byte < 4; ++byte) {
        const int i = 4 * w + byte;
        const uint32_t low = static_cast<uint32_t>(av >> (4 * i)) & 0xfu;
        const uint32_t high = static_cast<uint32_t>(bv >> (4 * i)) & 0xfu;
        word |= (low | (high << 4)) << (8 * byte);
      }
      out[w] = word;
    }
    reinterpret_cast<uint4*>(dst)[u] = make_uint4(out[0], out[1], out[2], out[3]);
  }
}

}  // namespace

int launch_repack(const uint8_t* state_bits, const uint8_t* w4_payload, const float* w4_scales,
                  const int8_t* w8_payload, const float* w8_scales, const int32_t* w4_row_offsets,
                  const int32_t* w8_row_offsets, int n_j, int n_k, void* prepared,
                  cudaStream_t stream) {
  const int64_t tiles = static_cast<int64_t>(n_j) * n_k;
  TileRecord* records = static_cast<TileRecord*>(prepared);
  uint8_t* payload = static_cast<uint8_t*>(prepared) + records_bytes(tiles);
  repack_kernel<<<static_cast<unsigned>(tiles), 256, 0, stream>>>(
      state_bits, w4_payload, w4_scales, w8_payload, w8_scales, w4_row_offsets, w8_row_offsets,
      n_k, records, payload);
  return check_cuda(cudaGetLastError(), "repack launch");
}

}  // namespace aq
