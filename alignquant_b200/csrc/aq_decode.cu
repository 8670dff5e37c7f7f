// Persistent decode kernel: packed W4/W8 x A8 GEMV/GEMM for at most 32 rows.
//
// At decode sizes a whole layer is a few microseconds of HBM traffic, so the kernel
// is built to keep one uninterrupted byte stream per SM.  The layer's tiles are
// stored in (j, k) order in the prepared image; that 1-D sequence of T tiles is cut
// into G equal contiguous ranges, one per CTA, one CTA per SM ("stream-K").  Each
// CTA's producer warp streams its range through a deep shared-memory ring with bulk
// asynchronous copies: one copy per weight tile and one 64-byte copy per activation
// row of that K64 block, all counted on the stage's mbarrier.  Weight copies of the
// first ring fill are issued before the grid dependency is resolved, so under
// programmatic dependent launch they overlap the tail of the preceding kernel.
// Eight consumer warps (8 output columns each) run the integer dot products on
// mma.sync.m16n8k32.s8 (aq_tile_math.cuh), several tiles per loop trip so that the
// waits, shared-memory loads and MMAs of neighbouring tiles overlap; the FP32
// accumulation still visits the tiles in increasing k.
//
// A CTA range may start and end in the middle of a tile row.  A row that lies entirely
// inside one range is finished by that CTA.  Otherwise each CTA writes its partial
// FP32 tile to a workspace slot and bumps the row's counter; the CTA that arrives last
// sums the slots in increasing-k order (so the result does not depend on arrival
// order), applies the inverse output transform and stores the row.  Counters return to
// zero, so the workspace only has to be zeroed once by its owner.  Nothing spins on
// another CTA.
//
// Arithmetic contract: per K64 tile, float(int32 dot) * (activation scale * tile
// scale), separately rounded multiply and add in increasing k inside a range
// (alignquant/kernels/cuda/linear.cu:956-963, 1296-1301); range partials are added in
// range order like the reference's split-K reducer (linear.cu:1339-1343).
#include <mutex>

#include "aq_common.cuh"
#include "aq_ptx.cuh"
#include "aq_tile_math.cuh"

namespace aq {

__device__ int g_decode_status = 0;

namespace {

struct DecodeParams {
  const int8_t* xq;
  const float* act_scales;
  const TileRecord* records;
  const uint8_t* payload;
  const int32_t* u_metadata;
  void* out;
  int32_t* acc_dump;
  float* partials;    // [2 * ctas][16 * MT][64]
  int32_t* counters;  // [n_j], zero between launches
  int64_t m;
  int64_t total_tiles;
  int n_j;
  int n_k;
  int ctas;
  int scale_mode;
  int out_dtype;
};

constexpr int kStages = 16;
constexpr int kConsumerWarps = 8;
constexpr int kConsumerThreads = kConsumerWarps * 32;
constexpr int kThreads = kConsumerThreads + 32;
constexpr int kXRowStride = 64;  // one K64 block of one activation row
constexpr int kMaxRecords = 1024;
constexpr int kNumBars = 2 * kStages;
constexpr int kMaxCounterRows = 16384;  // counters occupy a fixed region so that one workspace serves any layer
constexpr int64_t kCounterBytes = static_cast<int64_t>(kMaxCounterRows) * 4;

__host__ __device__ constexpr int stage_bytes(int mt) { return kW8TileBytes + 16 * mt * kXRowStride; }

__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, 256;" ::: "memory"); }

// first tile of CTA i, and the CTA that owns tile t, for T tiles cut into G ranges
__device__ __forceinline__ int64_t range_begin(int64_t i, int64_t total, int ctas) { return i * total / ctas; }
__device__ __forceinline__ int owner_of(int64_t t, int64_t total, int ctas) {
  return static_cast<int>(((t + 1) * ctas - 1) / total);
}

// Shared memory: [ring kStages x stage_bytes][tile 16*MT x 64 f32][records][barriers][flags]
template <int MT>
__global__ void __launch_bounds__(kThreads, 2) decode_linear_kernel(const DecodeParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  constexpr int kStage = stage_bytes(MT);
  constexpr int kRows = 16 * MT;
  uint8_t* ring = smem;
  float* tile = reinterpret_cast<float*>(smem + kStages * kStage);
  TileRecord* recs = reinterpret_cast<TileRecord*>(tile + kRows * kTile);
  uint64_t* bars = reinterpret_cast<uint64_t*>(recs + kMaxRecords);
  volatile uint32_t* abort_flag = reinterpret_cast<uint32_t*>(bars + kNumBars);
  volatile uint32_t* last_flag = abort_flag + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int n_k = p.n_k;
  const int64_t t0 = range_begin(blockIdx.x, p.total_tiles, p.ctas);
  const int64_t t1 = range_begin(blockIdx.x + 1, p.total_tiles, p.ctas);
  const int count = static_cast<int>(t1 - t0);
  const int rows = p.m < kRows ? static_cast<int>(p.m) : kRows;

  const uint32_t bar0 = smem_u32(bars);
  auto full = [&](int s) { return bar0 + 8u * s; };
  auto empty = [&](int s) { return bar0 + 8u * (kStages + s); };
  const uint32_t ring_addr = smem_u32(ring);

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(full(s), 1);
      mbar_init(empty(s), kConsumerWarps);
    }
    *abort_flag = 0;
    mbar_init_fence();
    fence_proxy_async();
  }
  __syncthreads();

  const TileRecord* my_records = p.records + t0;
  const bool producer = warp == kConsumerWarps;
  const uint32_t x_bytes = static_cast<uint32_t>(rows) * kTile;

  // First ring fill, weights only: they do not depend on the preceding kernel.
  if (producer && lane < kStages && lane < count) {
    const TileRecord r = my_records[lane];
    const uint32_t bytes = (r.offset_flag & kW4Flag) ? kW4TileBytes : kW8TileBytes;
    mbar_expect_tx(full(lane), bytes + x_bytes);
    bulk_copy(ring_addr + lane * kStage,
              p.payload + static_cast<int64_t>(r.offset_flag & ~kW4Flag) * kW4TileBytes, bytes, full(lane));
  }
  for (int i = threadIdx.x; i < count; i += kThreads) recs[i] = my_records[i];
  grid_launch_dependents();
  grid_dependency_wait();  // activations, scales, workspace and output belong to earlier kernels
  __syncthreads();

  if (producer) {
    const int64_t k_bytes = static_cast<int64_t>(n_k) * kTile;
    for (int i = 0; i < count; ++i) {
      const int s = i % kStages;
      int ok = 1;
      if (i >= kStages) {
        if (lane == 0) {
          ok = mbar_wait(empty(s), ((i / kStages) - 1) & 1, abort_flag, &g_decode_status, 21) ? 1 : 0;
          if (ok) {
            const TileRecord r = recs[i];
            const uint32_t bytes = (r.offset_flag & kW4Flag) ? kW4TileBytes : kW8TileBytes;
            mbar_expect_tx(full(s), bytes + x_bytes);
            bulk_copy(ring_addr + s * kStage,
                      p.payload + static_cast<int64_t>(r.offset_flag & ~kW4Flag) * kW4TileBytes, bytes, full(s));
          }
        }
        ok = __shfl_sync(0xffffffffu, ok, 0);
      }
      if (!ok) break;
      const int kt = static_cast<int>((t0 + i) % n_k);
      if (lane < rows) {
        bulk_copy(ring_addr + s * kStage + kW8TileBytes + lane * kXRowStride,
                  p.xq + lane * k_bytes + static_cast<int64_t>(kt) * kTile, kTile, full(s));
      }
    }
    return;
  }

  // ---- consumers: warp w owns output columns 8w .. 8w+7 --------------------------------
  const int g = lane >> 2;
  const int c = lane & 3;
  const int n = warp * 8 + g;
  constexpr int kUnroll = MT == 1 ? 4 : 2;
  float token_scale[MT][2];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) {
    const int r_lo = mt * 16 + g;
    token_scale[mt][0] = (p.scale_mode == AQ_SCALE_TOKEN && r_lo < rows) ? p.act_scales[r_lo] : 0.0f;
    token_scale[mt][1] = (p.scale_mode == AQ_SCALE_TOKEN && r_lo + 8 < rows) ? p.act_scales[r_lo + 8] : 0.0f;
  }
  const int64_t n_cols = static_cast<int64_t>(p.n_j) * kTile;

  int i = 0;
  bool ok = true;
  while (i < count && ok) {
    const int64_t t_first = t0 + i;
    const int j = static_cast<int>(t_first / n_k);
    const int k_lo = static_cast<int>(t_first - static_cast<int64_t>(j) * n_k);
    const int64_t row_end = static_cast<int64_t>(j + 1) * n_k;
    const int seg_tiles = static_cast<int>((row_end < t1 ? row_end : t1) - t_first);
    const bool whole_row = k_lo == 0 && seg_tiles == n_k;
    const int seg_begin = i;

    float acc[MT][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
      for (int q = 0; q < 4; ++q) acc[mt][q] = 0.0f;
    }
    const int seg_end = i + seg_tiles;
    while (i < seg_end && ok) {
      const int batch = seg_end - i < kUnroll ? seg_end - i : kUnroll;
      TileRecord rec[kUnroll];
      int d[kUnroll][MT][4];
      // waits first, then every load, then every MMA: independent chains the scheduler can overlap
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        if (u < batch && ok) {
          ok = mbar_wait(full((i + u) % kStages), ((i + u) / kStages) & 1, abort_flag, &g_decode_status, 22);
        }
      }
      if (!ok) break;
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        if (u < batch) {
          rec[u] = recs[i + u];
          const uint8_t* stage = ring + ((i + u) % kStages) * kStage;
          const uint4 w = load_weight_vector(stage, (rec[u].offset_flag & kW4Flag) != 0, n, c);
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
            const int r_lo = mt * 16 + g;
            uint4 x_lo = make_uint4(0, 0, 0, 0), x_hi = make_uint4(0, 0, 0, 0);
            const uint8_t* xp = stage + kW8TileBytes + r_lo * kXRowStride + c * 16;
            if (r_lo < rows) x_lo = *reinterpret_cast<const uint4*>(xp);
            if (r_lo + 8 < rows) x_hi = *reinterpret_cast<const uint4*>(xp + 8 * kXRowStride);
            tile_dot(d[u][mt], x_lo, x_hi, w);
          }
        }
      }
      // every lane's operands have been consumed by the warp-wide MMAs above
      __syncwarp();
      if (lane == 0) {
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
          if (u < batch && i + u + kStages < count) mbar_arrive(empty((i + u) % kStages));
        }
      }
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        if (u < batch) {
          const int kt = k_lo + (i + u - seg_begin);
          const bool is_w4 = (rec[u].offset_flag & kW4Flag) != 0;
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
            float s_lo, s_hi;
            if (p.scale_mode == AQ_SCALE_TOKEN) {
              s_lo = __fmul_rn(token_scale[mt][0], rec[u].scale);
              s_hi = __fmul_rn(token_scale[mt][1], rec[u].scale);
            } else {
              const float a_s = (mt * 16 < rows) ? p.act_scales[static_cast<int64_t>(mt) * n_k + kt] : 0.0f;
              s_lo = s_hi = __fmul_rn(a_s, rec[u].scale);
            }
            tile_accumulate(acc[mt], d[u][mt], s_lo, s_hi);
            if (p.acc_dump != nullptr) {
              const int shift = is_w4 ? 4 : 0;
              const int col_out = warp * 8 + 2 * c;
              const int r_lo = mt * 16 + g;
              if (r_lo < rows) {
                int32_t* o = p.acc_dump + ((static_cast<int64_t>(r_lo) * p.n_j + j) * n_k + kt) * kTile + col_out;
                o[0] = d[u][mt][0] >> shift;
                o[1] = d[u][mt][1] >> shift;
              }
              if (r_lo + 8 < rows) {
                int32_t* o = p.acc_dump + ((static_cast<int64_t>(r_lo + 8) * p.n_j + j) * n_k + kt) * kTile + col_out;
                o[0] = d[u][mt][2] >> shift;
                o[1] = d[u][mt][3] >> shift;
              }
            }
          }
        }
      }
      i += batch;
    }
    if (!ok) break;

    // ---- finish the segment ------------------------------------------------------------
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
      const int col = warp * 8 + 2 * c;
      *reinterpret_cast<float2*>(&tile[(mt * 16 + g) * kTile + col]) = make_float2(acc[mt][0], acc[mt][1]);
      *reinterpret_cast<float2*>(&tile[(mt * 16 + g + 8) * kTile + col]) = make_float2(acc[mt][2], acc[mt][3]);
    }
    consumer_sync();
    const int32_t* meta = p.u_metadata ? p.u_metadata + static_cast<int64_t>(j) * 4 * kTile : nullptr;
    const bool has_u = meta != nullptr && meta[0] != 0;
    int first_cta = blockIdx.x, last_cta = blockIdx.x;
    bool finish = whole_row;
    if (!whole_row) {
      // partial: publish to the workspace; the last arriver of the row finishes it
      const int slot = 2 * blockIdx.x + (seg_begin == 0 ? 0 : 1);  // 0: first segment of this CTA
      float* dst = p.partials + static_cast<int64_t>(slot) * kRows * kTile;
      for (int e = threadIdx.x; e < rows * kTile; e += kConsumerThreads) __stcg(dst + e, tile[e]);
      __threadfence();
      consumer_sync();
      first_cta = owner_of(static_cast<int64_t>(j) * n_k, p.total_tiles, p.ctas);
      last_cta = owner_of(row_end - 1, p.total_tiles, p.ctas);
      if (threadIdx.x == 0) {
        const int arrived = atomicAdd(p.counters + j, 1);
        const bool last = arrived == last_cta - first_cta;
        if (last) p.counters[j] = 0;  // every contributor has arrived: safe to reset
        *last_flag = last ? 1u : 0u;
      }
      consumer_sync();
      finish = *last_flag != 0;
      if (finish) __threadfence();
    }
    if (finish) {
      for (int row = warp; row < rows; row += kConsumerWarps) {
        float lo, hi;
        if (whole_row) {
          lo = tile[row * kTile + lane];
          hi = tile[row * kTile + lane + 32];
        } else {
          lo = hi = 0.0f;
          for (int cta = first_cta; cta <= last_cta; ++cta) {
            // a CTA's first segment sits in slot 0, any later one in slot 1
            const int64_t cta_begin = range_begin(cta, p.total_tiles, p.ctas);
            const int which = (cta_begin >= static_cast<int64_t>(j) * n_k) ? 0 : 1;
            const float* src = p.partials + (static_cast<int64_t>(2 * cta + which) * kRows + row) * kTile;
            const float a = __ldcg(src + lane);
            const float b = __ldcg(src + lane + 32);
            lo = (cta == first_cta) ? a : __fadd_rn(lo, a);
            hi = (cta == first_cta) ? b : __fadd_rn(hi, b);
          }
        }
        if (has_u) inverse_u_row(lo, hi, meta, lane);
        const int64_t o = static_cast<int64_t>(row) * n_cols + static_cast<int64_t>(j) * kTile + lane;
        store_any(p.out, p.out_dtype, o, lo);
        store_any(p.out, p.out_dtype, o + 32, hi);
      }
    }
    consumer_sync();  // the tile and the last-arriver flag are reused by the next segment
  }
}

int smem_bytes(int mt) {
  return kStages * stage_bytes(mt) + 16 * mt * kTile * 4 + kMaxRecords * 8 + kNumBars * 8 + 16;
}

template <int MT>
int launch_mt(const DecodeParams& p, cudaStream_t stream) {
  static std::once_flag once[64];
  int device = 0;
  int rc = check_cuda(cudaGetDevice(&device), "cudaGetDevice");
  if (rc != AQ_OK) return rc;
  cudaError_t attr_status = cudaSuccess;
  std::call_once(once[device & 63], [&] {
    attr_status = cudaFuncSetAttribute(decode_linear_kernel<MT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       smem_bytes(MT));
  });
  rc = check_cuda(attr_status, "cudaFuncSetAttribute(decode_linear_kernel)");
  if (rc != AQ_OK) return rc;
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(static_cast<unsigned>(p.ctas), 1, 1);
  config.blockDim = dim3(kThreads, 1, 1);
  config.dynamicSmemBytes = static_cast<size_t>(smem_bytes(MT));
  config.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attr;
  config.numAttrs = use_dependent_launch() ? 1 : 0;
  return check_cuda(cudaLaunchKernelEx(&config, decode_linear_kernel<MT>, p), "decode linear launch");
}

int64_t partial_bytes(int ctas, int mt) { return 2LL * ctas * 16 * mt * kTile * 4; }

}  // namespace

int decode_ctas(int n_j, int n_k) {
  const int64_t total = static_cast<int64_t>(n_j) * n_k;
  const int64_t sms = num_sms();
  int64_t ctas = sms;
  while ((total + ctas - 1) / ctas > kMaxRecords) ctas += sms;
  return static_cast<int>(total < ctas ? total : ctas);
}

int64_t decode_workspace_bytes(int64_t m, int n_j, int n_k) {
  const int mt = m <= 16 ? 1 : 2;
  return kCounterBytes + partial_bytes(decode_ctas(n_j, n_k), mt);
}

int launch_decode_linear(const LinearArgs& a, cudaStream_t stream) {
  if (a.n_j > kMaxCounterRows) {
    return fail(AQ_ERR_INVALID, "the decode kernel supports N up to %d, got %d", kMaxCounterRows * kTile, a.n_j * kTile);
  }
  DecodeParams p;
  p.xq = a.xq;
  p.act_scales = a.act_scales;
  p.records = a.records;
  p.payload = a.payload;
  p.u_metadata = a.u_metadata;
  p.out = a.out;
  p.acc_dump = a.acc_dump;
  p.counters = static_cast<int32_t*>(a.workspace);
  p.partials = reinterpret_cast<float*>(static_cast<uint8_t*>(a.workspace) + kCounterBytes);
  p.m = a.m;
  p.total_tiles = static_cast<int64_t>(a.n_j) * a.n_k;
  p.n_j = a.n_j;
  p.n_k = a.n_k;
  p.ctas = decode_ctas(a.n_j, a.n_k);
  p.scale_mode = a.scale_mode;
  p.out_dtype = a.out_dtype;
  return a.m <= 16 ? launch_mt<1>(p, stream) : launch_mt<2>(p, stream);
}

int take_decode_status() {
  int status = 0;
  if (cudaMemcpyFromSymbol(&status, g_decode_status, sizeof(int)) != cudaSuccess) return -1;
  if (status != 0) {
    const int zero = 0;
    cudaMemcpyToSymbol(g_decode_status, &zero, sizeof(int));
  }
  return status;
}

}  // namespace aq
