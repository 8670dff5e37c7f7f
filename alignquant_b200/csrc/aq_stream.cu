// Streaming mixed W4/W8 x A8 kernel for small row counts (decode and short prefill).
//
// The layer is bound by weight bytes here, so the kernel is organised around the
// HBM stream: a CTA owns one 64-column output tile row j and one K range (split),
// its 8 warps each own 8 of the 64 columns, and every lane issues exactly one
// 128-bit load per weight tile (W8: 16 consecutive k of one column; W4: 32 k of one
// column packed two per byte), kept PREFETCH tiles ahead in registers.  The integer
// dot products run on mma.sync.m16n8k32.s8 so that 1..16 rows cost the same; W4
// nibbles are widened with one shift and one mask to 16*w (the factor 1/16 is folded
// into the tile scale, which is exact).  Each K64 tile's int32 result is converted
// to FP32, multiplied by (activation scale * tile scale) and added to an FP32
// accumulator with separately rounded multiply and add, in increasing k -- the
// operation order of the reference kernels (alignquant/kernels/cuda/linear.cu:
// 956-963, 1296-1301).  Split-K partial tiles are exchanged through distributed
// shared memory of a thread-block cluster and summed in split order (the order of
// the reference reducer, linear.cu:1339-1343): no workspace, no second launch, no
// atomics.  The inverse output transform follows linear.cu:404-430.
#include <cooperative_groups.h>

#include "aq_common.cuh"

namespace cg = cooperative_groups;

namespace aq {
namespace {

struct StreamParams {
  const int8_t* xq;
  const float* act_scales;
  const TileRecord* records;
  const uint8_t* payload;
  const int32_t* u_metadata;
  void* out;
  int32_t* acc_dump;
  int64_t m;
  int n_j;
  int n_k;
  int scale_mode;
  int out_dtype;
};

constexpr int kPrefetch = 6;
constexpr int kMaxRecords = 512;  // records of one CTA's K range kept in shared memory

__device__ __forceinline__ uint4 ldg_stream(const uint8_t* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

__device__ __forceinline__ void mma_s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                       uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
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

template <int MT>
__global__ void __launch_bounds__(256) stream_linear_kernel(const StreamParams p) {
  __shared__ TileRecord rec_smem[kMaxRecords];
  __shared__ __align__(16) float tile[MT * 16][kTile];

  cg::cluster_group cluster = cg::this_cluster();
  const int split_k = static_cast<int>(cluster.num_blocks());
  const int split = static_cast<int>(cluster.block_rank());
  const int j = blockIdx.x;
  const int64_t m0 = static_cast<int64_t>(blockIdx.z) * (MT * 16);
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int g = lane >> 2;
  const int c = lane & 3;
  const int n_k = p.n_k;
  const int64_t k_bytes = static_cast<int64_t>(n_k) * kTile;
  const int k_begin = static_cast<int>(static_cast<int64_t>(n_k) * split / split_k);
  const int k_end = static_cast<int>(static_cast<int64_t>(n_k) * (split + 1) / split_k);
  const int k_count = k_end - k_begin;

  const TileRecord* row_records = p.records + static_cast<int64_t>(j) * n_k + k_begin;
  const bool records_in_smem = k_count <= kMaxRecords;
  if (records_in_smem) {
    for (int i = threadIdx.x; i < k_count; i += 256) rec_smem[i] = row_records[i];
  }
  __syncthreads();
  const TileRecord* recs = records_in_smem ? rec_smem : row_records;

  // per-lane byte offsets inside a tile
  const uint32_t lane_off_w8 = static_cast<uint32_t>((c * 8 + warp) * 128 + g * 16);
  const uint32_t lane_off_w4 = static_cast<uint32_t>(((c >> 1) * 8 + warp) * 128 + g * 16);
  const int w4_shift = (c & 1) ? 0 : 4;

  float acc[MT][4];
  float token_scale[MT][2];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[mt][i] = 0.0f;
    const int64_t r_lo = m0 + mt * 16 + g;
    token_scale[mt][0] = (p.scale_mode == AQ_SCALE_TOKEN && r_lo < p.m) ? p.act_scales[r_lo] : 0.0f;
    token_scale[mt][1] =
        (p.scale_mode == AQ_SCALE_TOKEN && r_lo + 8 < p.m) ? p.act_scales[r_lo + 8] : 0.0f;
  }

  uint4 wbuf[kPrefetch];
  TileRecord rbuf[kPrefetch];

  auto issue = [&](int slot_kt, uint4& w, TileRecord& r) {
    r = recs[slot_kt - k_begin];
    const bool is_w4 = (r.offset_flag & kW4Flag) != 0;
    const uint8_t* base =
        p.payload + static_cast<int64_t>(r.offset_flag & ~kW4Flag) * kW4TileBytes;
    w = ldg_stream(base + (is_w4 ? lane_off_w4 : lane_off_w8));
  };

#pragma unroll
  for (int u = 0; u < kPrefetch; ++u) {
    if (k_begin + u < k_end) issue(k_begin + u, wbuf[u], rbuf[u]);
  }

  for (int base_kt = k_begin; base_kt < k_end; base_kt += kPrefetch) {
#pragma unroll
    for (int u = 0; u < kPrefetch; ++u) {
      const int kt = base_kt + u;
      if (kt < k_end) {
        uint4 w = wbuf[u];
        const TileRecord r = rbuf[u];
        const bool is_w4 = (r.offset_flag & kW4Flag) != 0;
        if (kt + kPrefetch < k_end) issue(kt + kPrefetch, wbuf[u], rbuf[u]);
        if (is_w4) {
          w.x = (w.x << w4_shift) & 0xf0f0f0f0u;
          w.y = (w.y << w4_shift) & 0xf0f0f0f0u;
          w.z = (w.z << w4_shift) & 0xf0f0f0f0u;
          w.w = (w.w << w4_shift) & 0xf0f0f0f0u;
        }
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
          const int64_t r_lo = m0 + mt * 16 + g;
          const int64_t r_hi = r_lo + 8;
          uint4 a_lo = make_uint4(0, 0, 0, 0), a_hi = make_uint4(0, 0, 0, 0);
          const int64_t col = static_cast<int64_t>(kt) * kTile + c * 16;
          if (r_lo < p.m) a_lo = *reinterpret_cast<const uint4*>(p.xq + r_lo * k_bytes + col);
          if (r_hi < p.m) a_hi = *reinterpret_cast<const uint4*>(p.xq + r_hi * k_bytes + col);
          int d[4] = {0, 0, 0, 0};
          mma_s8(d, a_lo.x, a_hi.x, a_lo.y, a_hi.y, w.x, w.y);
          mma_s8(d, a_lo.z, a_hi.z, a_lo.w, a_hi.w, w.z, w.w);
          float s_lo, s_hi;
          if (p.scale_mode == AQ_SCALE_TOKEN) {
            s_lo = __fmul_rn(token_scale[mt][0], r.scale);
            s_hi = __fmul_rn(token_scale[mt][1], r.scale);
          } else {
            const int64_t mtile = (m0 >> 4) + mt;
            const float a_s = (mtile * 16 < p.m) ? p.act_scales[mtile * n_k + kt] : 0.0f;
            s_lo = s_hi = __fmul_rn(a_s, r.scale);
          }
          acc[mt][0] = __fadd_rn(acc[mt][0], __fmul_rn(static_cast<float>(d[0]), s_lo));
          acc[mt][1] = __fadd_rn(acc[mt][1], __fmul_rn(static_cast<float>(d[1]), s_lo));
          acc[mt][2] = __fadd_rn(acc[mt][2], __fmul_rn(static_cast<float>(d[2]), s_hi));
          acc[mt][3] = __fadd_rn(acc[mt][3], __fmul_rn(static_cast<float>(d[3]), s_hi));
          if (p.acc_dump != nullptr) {
            const int shift = is_w4 ? 4 : 0;
            const int col_out = warp * 8 + 2 * c;
            if (r_lo < p.m) {
              int32_t* o = p.acc_dump + ((r_lo * p.n_j + j) * n_k + kt) * kTile + col_out;
              o[0] = d[0] >> shift;
              o[1] = d[1] >> shift;
            }
            if (r_hi < p.m) {
              int32_t* o = p.acc_dump + ((r_hi * p.n_j + j) * n_k + kt) * kTile + col_out;
              o[0] = d[2] >> shift;
              o[1] = d[3] >> shift;
            }
          }
        }
      }
    }
  }

  // ---- split-K exchange through cluster shared memory --------------------------
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) {
    const int col = warp * 8 + 2 * c;
    *reinterpret_cast<float2*>(&tile[mt * 16 + g][col]) = make_float2(acc[mt][0], acc[mt][1]);
    *reinterpret_cast<float2*>(&tile[mt * 16 + g + 8][col]) = make_float2(acc[mt][2], acc[mt][3]);
  }
  cluster.sync();

  const int64_t rows_left = p.m - m0;
  const int rows = rows_left < MT * 16 ? static_cast<int>(rows_left) : MT * 16;
  const int32_t* meta =
      p.u_metadata ? p.u_metadata + static_cast<int64_t>(j) * 4 * kTile : nullptr;
  const bool has_u = meta != nullptr && meta[0] != 0;
  const int64_t n_cols = static_cast<int64_t>(p.n_j) * kTile;
  // rank r finishes rows r, r + split_k, ...; its warps take them round robin
  for (int row = split + split_k * warp; row < rows; row += split_k * 8) {
    float lo = 0.0f, hi = 0.0f;
    for (int s = 0; s < split_k; ++s) {
      const float* remote = cluster.map_shared_rank(&tile[0][0], s);
      const float a = remote[row * kTile + lane];
      const float b = remote[row * kTile + lane + 32];
      lo = (s == 0) ? a : __fadd_rn(lo, a);
      hi = (s == 0) ? b : __fadd_rn(hi, b);
    }
    if (has_u) inverse_u_row(lo, hi, meta, lane);
    const int64_t o = (m0 + row) * n_cols + static_cast<int64_t>(j) * kTile + lane;
    store_any(p.out, p.out_dtype, o, lo);
    store_any(p.out, p.out_dtype, o + 32, hi);
  }
  cluster.sync();  // peers may still be reading this CTA's tile
}

template <int MT>
int launch_mt(const StreamParams& p, int split_k, cudaStream_t stream) {
  const int64_t m_blocks = (p.m + MT * 16 - 1) / (MT * 16);
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(static_cast<unsigned>(p.n_j), static_cast<unsigned>(split_k),
                        static_cast<unsigned>(m_blocks));
  config.blockDim = dim3(256, 1, 1);
  config.dynamicSmemBytes = 0;
  config.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = static_cast<unsigned>(split_k);
  attr[0].val.clusterDim.z = 1;
  config.attrs = attr;
  config.numAttrs = 1;
  return check_cuda(cudaLaunchKernelEx(&config, stream_linear_kernel<MT>, p),
                    "streaming linear launch");
}

}  // namespace

int stream_auto_split(int64_t m, int n_j, int n_k) {
  const int64_t rows_per_cta = m <= 16 ? 16 : (m <= 32 ? 32 : (m <= 64 ? 64 : 128));
  const int64_t m_blocks = (m + rows_per_cta - 1) / rows_per_cta;
  const int64_t target = 2LL * num_sms();
  int split = 1;
  while (split < 8 && static_cast<int64_t>(n_j) * m_blocks * split < target &&
         n_k / (2 * split) >= 4) {
    split *= 2;
  }
  return split;
}

int launch_stream_linear(const LinearArgs& a, int split_k, cudaStream_t stream) {
  StreamParams p;
  p.xq = a.xq;
  p.act_scales = a.act_scales;
  p.records = a.records;
  p.payload = a.payload;
  p.u_metadata = a.u_metadata;
  p.out = a.out;
  p.acc_dump = a.acc_dump;
  p.m = a.m;
  p.n_j = a.n_j;
  p.n_k = a.n_k;
  p.scale_mode = a.scale_mode;
  p.out_dtype = a.out_dtype;
  if (split_k < 1) split_k = 1;
  if (split_k > 8) split_k = 8;
  while (split_k > a.n_k) split_k /= 2;
  if (a.m <= 16) return launch_mt<1>(p, split_k, stream);
  if (a.m <= 32) return launch_mt<2>(p, split_k, stream);
  if (a.m <= 64) return launch_mt<4>(p, split_k, stream);
  return launch_mt<8>(p, split_k, stream);
}

}  // namespace aq
