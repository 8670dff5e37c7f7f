// Streaming mixed W4/W8 x A8 kernel for small row counts (decode and short prefill).
//
// The layer is bound by weight bytes here, so the kernel is organised around the HBM
// stream.  A CTA owns one 64-column output tile row j, one K range (split) and up to
// 16*MT activation rows.  A producer warp streams the CTA's weight tiles from the
// prepared image into a shared-memory ring with one bulk asynchronous copy per tile
// (cp.async.bulk, completion counted on an mbarrier) and stages the CTA's slice of
// the int8 activations once.  Eight consumer warps, one per 8 output columns, read
// their operands with conflict-free 16-byte shared-memory loads and run the integer
// dot products on mma.sync.m16n8k32.s8, so 1..16 rows cost the same (aq_tile_math.cuh);
// W4 nibbles are widened with one shift and one mask to 16*w (the factor 1/16 is
// folded into the tile scale, which is exact).
//
// Each K64 tile's int32 result is converted to FP32, multiplied by
// (activation scale * tile scale) and added to an FP32 accumulator with separately
// rounded multiply and add, in increasing k -- the operation order of the reference
// kernels (alignquant/kernels/cuda/linear.cu:956-963, 1296-1301).  Split-K partial
// tiles are exchanged through distributed shared memory of a thread-block cluster and
// summed in split order (the order of the reference reducer, linear.cu:1339-1343): no
// workspace, no second launch, no atomics.  The inverse output transform follows
// linear.cu:404-430.  Every mbarrier wait is bounded (see aq_ptx.cuh).
#include <cooperative_groups.h>

#include <mutex>

#include "aq_common.cuh"
#include "aq_ptx.cuh"
#include "aq_tile_math.cuh"

namespace cg = cooperative_groups;

namespace aq {

__device__ int g_stream_status = 0;

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
  int x_stride;  // bytes between staged activation rows, congruent to 64 modulo 128
};

constexpr int kStages = 8;
constexpr int kConsumerWarps = 8;
constexpr int kThreads = (kConsumerWarps + 1) * 32;
constexpr int kMaxCount = 512;             // tiles of one CTA's K range
constexpr int kMaxXBytes = 96 * 1024;      // staged activation slice
constexpr int kNumBars = 2 * kStages + 1;  // full[], empty[], x_full
constexpr int kBarRegionBytes = (kNumBars + 3) * 8;  // barriers, abort flag, padding to 16 bytes

// Shared memory: [ring kStages x 4096][tile MT*16 x 64 f32][records k_count x 8]
//                [barriers][abort flag][activation slice rows x x_stride]
template <int MT>
__global__ void __launch_bounds__(kThreads) stream_linear_kernel(const StreamParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  uint8_t* ring = smem;
  float* tile = reinterpret_cast<float*>(smem + kStages * kW8TileBytes);
  TileRecord* recs = reinterpret_cast<TileRecord*>(tile + MT * 16 * kTile);

  cg::cluster_group cluster = cg::this_cluster();
  const int split_k = static_cast<int>(cluster.num_blocks());
  const int split = static_cast<int>(cluster.block_rank());
  const int j = blockIdx.x;
  const int64_t m0 = static_cast<int64_t>(blockIdx.z) * (MT * 16);
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int n_k = p.n_k;
  const int k_begin = static_cast<int>(static_cast<int64_t>(n_k) * split / split_k);
  const int k_end = static_cast<int>(static_cast<int64_t>(n_k) * (split + 1) / split_k);
  const int k_count = k_end - k_begin;
  const int64_t rows_left = p.m - m0;
  const int rows = rows_left < MT * 16 ? static_cast<int>(rows_left) : MT * 16;

  uint64_t* bars = reinterpret_cast<uint64_t*>(recs + ((k_count + 1) & ~1));
  volatile uint32_t* abort_flag = reinterpret_cast<uint32_t*>(bars + kNumBars);
  uint8_t* xs = reinterpret_cast<uint8_t*>(bars) + kBarRegionBytes;  // 16-byte aligned
  const uint32_t bar0 = smem_u32(bars);
  auto full = [&](int s) { return bar0 + 8u * s; };
  auto empty = [&](int s) { return bar0 + 8u * (kStages + s); };
  const uint32_t x_full = bar0 + 8u * (2 * kStages);
  const uint32_t ring_addr = smem_u32(ring);

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(full(s), 1);
      mbar_init(empty(s), kConsumerWarps);
    }
    mbar_init(x_full, 1);
    *abort_flag = 0;
    mbar_init_fence();
    fence_proxy_async();
  }
  __syncthreads();

  const TileRecord* row_records = p.records + static_cast<int64_t>(j) * n_k + k_begin;
  const bool producer = warp == kConsumerWarps;

  // Weights do not depend on the preceding kernel: the first ring fill is issued before
  // the grid dependency is resolved, one tile per producer lane.
  if (producer && lane < kStages && lane < k_count) {
    const TileRecord r = row_records[lane];
    const uint32_t bytes = (r.offset_flag & kW4Flag) ? kW4TileBytes : kW8TileBytes;
    mbar_expect_tx(full(lane), bytes);
    bulk_copy(ring_addr + lane * kW8TileBytes,
              p.payload + static_cast<int64_t>(r.offset_flag & ~kW4Flag) * kW4TileBytes, bytes, full(lane));
  }
  for (int i = threadIdx.x; i < k_count; i += kThreads) recs[i] = row_records[i];
  grid_launch_dependents();
  grid_dependency_wait();  // activations and their scales come from the preceding kernel
  __syncthreads();

  float acc[MT][4];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[mt][i] = 0.0f;
  }

  if (producer) {
    // ---- activation slice: one bulk copy per valid row --------------------------
    const uint32_t row_bytes = static_cast<uint32_t>(k_count) * kTile;
    if (lane == 0) mbar_expect_tx(x_full, row_bytes * rows);
    __syncwarp();
    for (int r = lane; r < rows; r += 32) {
      bulk_copy(smem_u32(xs) + r * p.x_stride,
                p.xq + (m0 + r) * (static_cast<int64_t>(n_k) * kTile) + static_cast<int64_t>(k_begin) * kTile,
                row_bytes, x_full);
    }
    // ---- ring refills ---------------------------------------------------------------
    if (lane == 0) {
      for (int i = kStages; i < k_count; ++i) {
        const int s = i % kStages;
        if (!mbar_wait(empty(s), ((i / kStages) - 1) & 1, abort_flag, &g_stream_status, 11)) break;
        const TileRecord r = recs[i];
        const uint32_t bytes = (r.offset_flag & kW4Flag) ? kW4TileBytes : kW8TileBytes;
        mbar_expect_tx(full(s), bytes);
        bulk_copy(ring_addr + s * kW8TileBytes,
                  p.payload + static_cast<int64_t>(r.offset_flag & ~kW4Flag) * kW4TileBytes, bytes, full(s));
      }
    }
    __syncwarp();
  } else {
    // ---- consumers: warp w owns output columns 8w .. 8w+7 ---------------------------
    const int g = lane >> 2;
    const int c = lane & 3;
    const int n = warp * 8 + g;
    float token_scale[MT][2];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
      const int64_t r_lo = m0 + mt * 16 + g;
      token_scale[mt][0] = (p.scale_mode == AQ_SCALE_TOKEN && r_lo < p.m) ? p.act_scales[r_lo] : 0.0f;
      token_scale[mt][1] =
          (p.scale_mode == AQ_SCALE_TOKEN && r_lo + 8 < p.m) ? p.act_scales[r_lo + 8] : 0.0f;
    }
    bool ok = mbar_wait(x_full, 0, abort_flag, &g_stream_status, 12);
    for (int i = 0; i < k_count && ok; ++i) {
      const int s = i % kStages;
      const int kt = k_begin + i;
      if (!mbar_wait(full(s), (i / kStages) & 1, abort_flag, &g_stream_status, 13)) break;
      const TileRecord r = recs[i];
      const bool is_w4 = (r.offset_flag & kW4Flag) != 0;
      const uint4 w = load_weight_vector(ring + s * kW8TileBytes, is_w4, n, c);
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        const int r_lo = mt * 16 + g;
        const int r_hi = r_lo + 8;
        uint4 x_lo = make_uint4(0, 0, 0, 0), x_hi = make_uint4(0, 0, 0, 0);
        const uint8_t* xp = xs + r_lo * p.x_stride + i * kTile + c * 16;
        if (r_lo < rows) x_lo = *reinterpret_cast<const uint4*>(xp);
        if (r_hi < rows) x_hi = *reinterpret_cast<const uint4*>(xp + 8 * p.x_stride);
        int d[4];
        tile_dot(d, x_lo, x_hi, w);
        float s_lo, s_hi;
        if (p.scale_mode == AQ_SCALE_TOKEN) {
          s_lo = __fmul_rn(token_scale[mt][0], r.scale);
          s_hi = __fmul_rn(token_scale[mt][1], r.scale);
        } else {
          const int64_t mtile = (m0 >> 4) + mt;
          const float a_s = (mtile * 16 < p.m) ? p.act_scales[mtile * n_k + kt] : 0.0f;
          s_lo = s_hi = __fmul_rn(a_s, r.scale);
        }
        tile_accumulate(acc[mt], d, s_lo, s_hi);
        if (p.acc_dump != nullptr) {
          const int shift = is_w4 ? 4 : 0;
          const int col_out = warp * 8 + 2 * c;
          if (r_lo < rows) {
            int32_t* o = p.acc_dump + (((m0 + r_lo) * p.n_j + j) * n_k + kt) * kTile + col_out;
            o[0] = d[0] >> shift;
            o[1] = d[1] >> shift;
          }
          if (r_hi < rows) {
            int32_t* o = p.acc_dump + (((m0 + r_hi) * p.n_j + j) * n_k + kt) * kTile + col_out;
            o[0] = d[2] >> shift;
            o[1] = d[3] >> shift;
          }
        }
      }
      // every lane's operand words have been consumed by the warp-wide MMAs above
      __syncwarp();
      if (lane == 0 && i + kStages < k_count) mbar_arrive(empty(s));
    }
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
      const int col = warp * 8 + 2 * c;
      *reinterpret_cast<float2*>(&tile[(mt * 16 + g) * kTile + col]) = make_float2(acc[mt][0], acc[mt][1]);
      *reinterpret_cast<float2*>(&tile[(mt * 16 + g + 8) * kTile + col]) = make_float2(acc[mt][2], acc[mt][3]);
    }
  }

  // ---- split-K exchange through cluster shared memory --------------------------------
  cluster.sync();
  if (!producer) {
    const int32_t* meta = p.u_metadata ? p.u_metadata + static_cast<int64_t>(j) * 4 * kTile : nullptr;
    const bool has_u = meta != nullptr && meta[0] != 0;
    const int64_t n_cols = static_cast<int64_t>(p.n_j) * kTile;
    // rank r finishes rows r, r + split_k, ...; its warps take them round robin
    for (int row = split + split_k * warp; row < rows; row += split_k * kConsumerWarps) {
      float lo = 0.0f, hi = 0.0f;
      for (int s = 0; s < split_k; ++s) {
        const float* remote = cluster.map_shared_rank(tile, s);
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
  }
  cluster.sync();  // peers may still be reading this CTA's tile
}

// bytes between staged activation rows: 64 * k_count rounded so that it is 64 modulo 128
int x_row_stride(int k_count) { return k_count * kTile + ((k_count & 1) ? 0 : kTile); }

int smem_bytes(int mt, int k_count, int rows) {
  return kStages * kW8TileBytes + mt * 16 * kTile * 4 + ((k_count + 1) & ~1) * 8 + kBarRegionBytes +
         rows * x_row_stride(k_count);
}

template <int MT>
int launch_mt(const StreamParams& p, int split_k, int k_count, cudaStream_t stream) {
  static std::once_flag once[64];
  int device = 0;
  int rc = check_cuda(cudaGetDevice(&device), "cudaGetDevice");
  if (rc != AQ_OK) return rc;
  cudaError_t attr_status = cudaSuccess;
  std::call_once(once[device & 63], [&] {
    attr_status = cudaFuncSetAttribute(stream_linear_kernel<MT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       200 * 1024);
  });
  rc = check_cuda(attr_status, "cudaFuncSetAttribute(stream_linear_kernel)");
  if (rc != AQ_OK) return rc;
  const int64_t m_blocks = (p.m + MT * 16 - 1) / (MT * 16);
  const int rows = p.m < MT * 16 ? static_cast<int>(p.m) : MT * 16;
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(static_cast<unsigned>(p.n_j), static_cast<unsigned>(split_k),
                        static_cast<unsigned>(m_blocks));
  config.blockDim = dim3(kThreads, 1, 1);
  config.dynamicSmemBytes = static_cast<size_t>(smem_bytes(MT, k_count, rows));
  config.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = static_cast<unsigned>(split_k);
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attr;
  config.numAttrs = use_dependent_launch() ? 2 : 1;
  return check_cuda(cudaLaunchKernelEx(&config, stream_linear_kernel<MT>, p), "streaming linear launch");
}

int rows_per_cta(int64_t m) { return m <= 16 ? 16 : (m <= 32 ? 32 : (m <= 64 ? 64 : 128)); }

}  // namespace

int stream_auto_split(int64_t m, int n_j, int n_k) {
  const int64_t rows = rows_per_cta(m);
  const int64_t m_blocks = (m + rows - 1) / rows;
  const int64_t target = 2LL * num_sms();
  int split = 1;
  while (split < 8 && static_cast<int64_t>(n_j) * m_blocks * split < target && n_k / (2 * split) >= 4) {
    split *= 2;
  }
  return split;
}

int launch_stream_linear(const LinearArgs& a, int split_k, cudaStream_t stream) {
  if (split_k < 1) split_k = 1;
  if (split_k > 8) split_k = 8;
  while (split_k > a.n_k) split_k /= 2;
  // rows per CTA: as many as the staged activation slice allows; more splits shorten it
  int rows = rows_per_cta(a.m);
  auto max_count = [&](int s) { return (a.n_k + s - 1) / s; };
  while (rows > 16 && static_cast<int64_t>(rows) * x_row_stride(max_count(split_k)) > kMaxXBytes) rows /= 2;
  while (split_k < 8 && split_k * 2 <= a.n_k &&
         (static_cast<int64_t>(rows) * x_row_stride(max_count(split_k)) > kMaxXBytes || max_count(split_k) > kMaxCount)) {
    split_k *= 2;
  }
  const int k_count = max_count(split_k);
  if (k_count > kMaxCount || static_cast<int64_t>(rows) * x_row_stride(k_count) > kMaxXBytes) {
    return fail(AQ_ERR_INVALID, "the streaming kernel supports K up to %d, got %d", 8 * kMaxXBytes / 16,
                a.n_k * kTile);
  }
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
  p.x_stride = x_row_stride(k_count);
  switch (rows) {
    case 16:
      return launch_mt<1>(p, split_k, k_count, stream);
    case 32:
      return launch_mt<2>(p, split_k, k_count, stream);
    case 64:
      return launch_mt<4>(p, split_k, k_count, stream);
    default:
      return launch_mt<8>(p, split_k, k_count, stream);
  }
}

int take_stream_status() {
  int status = 0;
  if (cudaMemcpyFromSymbol(&status, g_stream_status, sizeof(int)) != cudaSuccess) return -1;
  if (status != 0) {
    const int zero = 0;
    cudaMemcpyToSymbol(g_stream_status, &zero, sizeof(int));
  }
  return status;
}

}  // namespace aq
