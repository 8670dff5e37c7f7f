// Persistent decode kernel: packed W4/W8 x A8 GEMV/GEMM for at most 32 rows.
//
// At decode sizes a whole layer is a few microseconds of HBM traffic, so the kernel
// is built to keep one uninterrupted byte stream per SM.  The layer's tiles are
// stored in (j, k) order in the prepared image; that 1-D sequence of T tiles is cut
// into G equal contiguous ranges, one per CTA, one CTA per SM ("stream-K").  Each
// CTA's producer warp streams its range through a deep shared-memory ring with one
// bulk asynchronous copy per weight tile; four tiles share a ring slot and one
// full/empty mbarrier pair.  The copies of the first ring fill are issued before the
// grid dependency is resolved, so under programmatic dependent launch they overlap the
// tail of the preceding kernel.  Eight consumer warps (8 output columns each) run the
// integer dot products on mma.sync.m16n8k32.s8 (aq_tile_math.cuh) a slot at a time as
// straight-line code: activation vectors come from global memory (a few KiB, L1/L2
// resident) and are requested before the slot's barrier is waited on; the FP32
// accumulation still visits the tiles in increasing k.
//
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

#ifdef AQ_TRACE
// Development aid: timestamps of CTA 0 (consumer warp 0 and the producer), 4096 slots.
__device__ long long g_trace[4096];
#define AQ_TRACE_MARK(slot) \
  do { if (blockIdx.x == 0 && lane == 0 && (slot) < 4096) g_trace[(slot)] = clock64(); } while (0)
#else
#define AQ_TRACE_MARK(slot) do { } while (0)
#endif

namespace {

struct DecodeParams {
  const int8_t* xq;
  const float* act_scales;
  const TileRecord* records;
  const uint8_t* payload;
  const int32_t* u_metadata;
  void* out;
  int32_t* acc_dump;
  float* partials;    // [2 * ctas][8 * NT][64]
  int32_t* counters;  // [n_j], zero between launches
  int64_t m;
  int64_t total_tiles;
  int n_j;
  int n_k;
  int ctas;
  int scale_mode;
  int out_dtype;
};

constexpr int kGroupTiles = 8;  // tiles per ring slot: one full/empty barrier pair per slot
constexpr int kSlots = 3;       // ring depth in slots (24 tiles, 96 KiB)
constexpr int kSlotBytes = kGroupTiles * kW8TileBytes;
constexpr int kConsumerWarps = 4;  // 16 output columns each
constexpr int kConsumerThreads = kConsumerWarps * 32;
constexpr int kThreads = kConsumerThreads + 32;
constexpr int kMaxRecords = 1024;
constexpr int kNumBars = 2 * kSlots;
constexpr int kMaxCounterRows = 16384;  // counters occupy a fixed region so that one workspace serves any layer
constexpr int64_t kCounterBytes = static_cast<int64_t>(kMaxCounterRows) * 4;

__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

__device__ __forceinline__ uint4 ldg_x(const int8_t* p) {
  uint4 v;
  asm volatile("ld.global.nc.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

// first tile of CTA i, and the CTA that owns tile t, for T tiles cut into G ranges
__device__ __forceinline__ int64_t range_begin(int64_t i, int64_t total, int ctas) { return i * total / ctas; }
__device__ __forceinline__ int owner_of(int64_t t, int64_t total, int ctas) {
  return static_cast<int>(((t + 1) * ctas - 1) / total);
}

__device__ __forceinline__ uint32_t tile_bytes(const TileRecord& r) {
  return (r.offset_flag & kW4Flag) ? kW4TileBytes : kW8TileBytes;
}

// 16-byte weight vector of output column n, k in [16c, 16c+16), from a staged tile
// (layouts in aq_tile_math.cuh); W4 nibbles are widened to bytes holding 16*w.
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

// In this kernel the weights are the 16-row MMA operand (16 output columns per warp and
// MMA) and up to eight activation rows ("tokens") are the 8-column operand, so one pair
// of MMAs covers 16 columns x 8 tokens of a K64 tile.  Lane (g, c) = (lane/4, lane%4)
// holds the weight vectors of columns 16w+g and 16w+g+8 and the activation vector of
// token 8*pass+g, all for k in [16c, 16c+16).  Results: d[0], d[1] = column 16w+g,
// tokens 8*pass+2c, +1; d[2], d[3] = column 16w+g+8, same tokens.
//
// Shared memory: [ring kSlots x kGroupTiles x 4096][tile 8*NT x 64 f32][records][barriers][flags]
template <int NT>
__global__ void __launch_bounds__(kThreads, NT == 1 ? 2 : 1) decode_linear_kernel(const DecodeParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  constexpr int kRows = 8 * NT;
  uint8_t* ring = smem;
  float* tile = reinterpret_cast<float*>(smem + kSlots * kSlotBytes);
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
  const int groups = (count + kGroupTiles - 1) / kGroupTiles;
  const int rows = p.m < kRows ? static_cast<int>(p.m) : kRows;

  const uint32_t bar0 = smem_u32(bars);
  auto full = [&](int s) { return bar0 + 8u * s; };
  auto empty = [&](int s) { return bar0 + 8u * (kSlots + s); };
  const uint32_t ring_addr = smem_u32(ring);

  if (warp == 0) AQ_TRACE_MARK(4000);
  if (threadIdx.x == 0) {
    for (int s = 0; s < kSlots; ++s) {
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

  // First ring fill: weights do not depend on the preceding kernel, so these copies are
  // issued before the grid dependency is resolved.  Lane l fetches tile l of the range.
  if (producer) {
    constexpr int kFill = kSlots * kGroupTiles;
    static_assert(kFill <= 32 && kGroupTiles == 8, "the first fill uses one lane per tile");
    const bool active = lane < kFill && lane < count;
    TileRecord r = {0u, 0.0f};
    if (active) r = my_records[lane];
    const uint32_t bytes = active ? tile_bytes(r) : 0u;
    uint32_t group_bytes = bytes;
    group_bytes += __shfl_xor_sync(0xffffffffu, group_bytes, 1);
    group_bytes += __shfl_xor_sync(0xffffffffu, group_bytes, 2);
    group_bytes += __shfl_xor_sync(0xffffffffu, group_bytes, 4);
    if (active && (lane % kGroupTiles) == 0) mbar_expect_tx(full(lane / kGroupTiles), group_bytes);
    __syncwarp();
    if (active) {
      bulk_copy(ring_addr + lane * kW8TileBytes,
                p.payload + static_cast<int64_t>(r.offset_flag & ~kW4Flag) * kW4TileBytes, bytes,
                full(lane / kGroupTiles));
    }
  }
  for (int i = threadIdx.x; i < count; i += kThreads) recs[i] = my_records[i];
  grid_launch_dependents();
  grid_dependency_wait();  // activations, scales, workspace and output belong to earlier kernels
  __syncthreads();
  if (warp == 0) AQ_TRACE_MARK(4001);

  if (producer) {
    // ---- refills: one slot (up to eight tiles) per trip, lanes 0..7 issue the copies ----
    for (int gi = kSlots; gi < groups; ++gi) {
      const int slot = gi % kSlots;
      int ok = 1;
      if (lane == 0) {
        ok = mbar_wait(empty(slot), ((gi / kSlots) - 1) & 1, abort_flag, &g_decode_status, 21) ? 1 : 0;
      }
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) break;
      AQ_TRACE_MARK(2048 + 2 * gi);
      const int i = gi * kGroupTiles + lane;
      const bool active = lane < kGroupTiles && i < count;
      TileRecord r = {0u, 0.0f};
      if (active) r = recs[i];
      const uint32_t bytes = active ? tile_bytes(r) : 0u;
      uint32_t group_bytes = bytes;
      group_bytes += __shfl_xor_sync(0xffffffffu, group_bytes, 1);
      group_bytes += __shfl_xor_sync(0xffffffffu, group_bytes, 2);
      group_bytes += __shfl_xor_sync(0xffffffffu, group_bytes, 4);
      if (lane == 0) mbar_expect_tx(full(slot), group_bytes);
      __syncwarp();
      if (active) {
        bulk_copy(ring_addr + slot * kSlotBytes + lane * kW8TileBytes,
                  p.payload + static_cast<int64_t>(r.offset_flag & ~kW4Flag) * kW4TileBytes, bytes, full(slot));
      }
      AQ_TRACE_MARK(2048 + 2 * gi + 1);
    }
    return;
  }

  // ---- consumers: warp w owns output columns 16w .. 16w+15 -----------------------------
  const int g = lane >> 2;
  const int c = lane & 3;
  const int n_a = warp * 16 + g;  // second column of this lane is n_a + 8
  const int64_t k_bytes = static_cast<int64_t>(n_k) * kTile;
  // byte offsets of this lane's 16-byte weight vectors inside a staged W8 / W4 tile
  const uint32_t w8_off = static_cast<uint32_t>(n_a * 64 + ((c ^ ((n_a >> 1) & 3)) << 4));
  const uint32_t w4_off = static_cast<uint32_t>(n_a * 32 + (c >> 1) * 16);
  const int w4_shift = (c & 1) ? 0 : 4;
  // per-token activation scale of the two tokens this lane's results belong to
  float token_scale[NT][2];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    const int tok = nt * 8 + 2 * c;
    token_scale[nt][0] = (p.scale_mode == AQ_SCALE_TOKEN && tok < rows) ? p.act_scales[tok] : 0.0f;
    token_scale[nt][1] = (p.scale_mode == AQ_SCALE_TOKEN && tok + 1 < rows) ? p.act_scales[tok + 1] : 0.0f;
  }
  const int64_t n_cols = static_cast<int64_t>(p.n_j) * kTile;
  const int8_t* x_lane[NT];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) x_lane[nt] = p.xq + static_cast<int64_t>(nt * 8 + g) * k_bytes + c * 16;

  // running position inside the (j, k) grid
  int j = static_cast<int>(t0 / n_k);
  int kt = static_cast<int>(t0 - static_cast<int64_t>(j) * n_k);
  bool first_segment = true;
  int seg_k_lo = kt;
  float acc[NT][4];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
    for (int q = 0; q < 4; ++q) acc[nt][q] = 0.0f;
  }

  // Finish the segment [seg_k_lo, k_hi) of row j held in `acc`.
  auto flush = [&](int k_hi) {
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      const int tok = nt * 8 + 2 * c;
      tile[tok * kTile + n_a] = acc[nt][0];
      tile[(tok + 1) * kTile + n_a] = acc[nt][1];
      tile[tok * kTile + n_a + 8] = acc[nt][2];
      tile[(tok + 1) * kTile + n_a + 8] = acc[nt][3];
#pragma unroll
      for (int q = 0; q < 4; ++q) acc[nt][q] = 0.0f;
    }
    consumer_sync();
    const bool whole_row = seg_k_lo == 0 && k_hi == n_k;
    const int32_t* meta = p.u_metadata ? p.u_metadata + static_cast<int64_t>(j) * 4 * kTile : nullptr;
    const bool has_u = meta != nullptr && meta[0] != 0;
    int first_cta = blockIdx.x, last_cta = blockIdx.x;
    bool finish = whole_row;
    if (!whole_row) {
      // partial: publish to the workspace; the last arriver of the row finishes it
      const int slot = 2 * blockIdx.x + (first_segment ? 0 : 1);
      float* dst = p.partials + static_cast<int64_t>(slot) * kRows * kTile;
      for (int e = threadIdx.x; e < rows * kTile; e += kConsumerThreads) __stcg(dst + e, tile[e]);
      __threadfence();
      consumer_sync();
      first_cta = owner_of(static_cast<int64_t>(j) * n_k, p.total_tiles, p.ctas);
      last_cta = owner_of(static_cast<int64_t>(j + 1) * n_k - 1, p.total_tiles, p.ctas);
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
    first_segment = false;
  };

  for (int gi = 0; gi < groups; ++gi) {
    const int slot = gi % kSlots;
    const int base = gi * kGroupTiles;
    const int batch = count - base < kGroupTiles ? count - base : kGroupTiles;

    // (1) activations of the batch straight from global memory (a few KiB, L1/L2
    //     resident); requested before the wait so that their latency hides behind it
    uint4 x[kGroupTiles][NT];
    {
      int kk = kt;
#pragma unroll
      for (int u = 0; u < kGroupTiles; ++u) {
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          x[u][nt] = make_uint4(0, 0, 0, 0);
          if (u < batch && nt * 8 + g < rows) x[u][nt] = ldg_x(x_lane[nt] + static_cast<int64_t>(kk) * kTile);
        }
        if (++kk == n_k) kk = 0;
      }
    }
    // (2) the slot's weights
    if (warp == 0) AQ_TRACE_MARK(2 * gi);
    if (!mbar_wait(full(slot), (gi / kSlots) & 1, abort_flag, &g_decode_status, 22)) break;
    if (warp == 0) AQ_TRACE_MARK(2 * gi + 1);
    // (3) + (4) records, weight vectors and integer dot products of the batch
    TileRecord rec[kGroupTiles];
#pragma unroll
    for (int u = 0; u < kGroupTiles; ++u) rec[u] = recs[base + (u < batch ? u : 0)];
    int d[kGroupTiles][NT][4];
#pragma unroll
    for (int u = 0; u < kGroupTiles; ++u) {
      const bool is_w4 = (rec[u].offset_flag & kW4Flag) != 0;
      const uint8_t* staged = ring + slot * kSlotBytes + u * kW8TileBytes;
      const uint4 wa = weight_vector(staged, is_w4, w8_off, w4_off, w4_shift);
      const uint4 wb = weight_vector(staged + (is_w4 ? 8 * 32 : 8 * 64), is_w4, w8_off, w4_off, w4_shift);
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        d[u][nt][0] = d[u][nt][1] = d[u][nt][2] = d[u][nt][3] = 0;
        mma_s8(d[u][nt], wa.x, wb.x, wa.y, wb.y, x[u][nt].x, x[u][nt].y);
        mma_s8(d[u][nt], wa.z, wb.z, wa.w, wb.w, x[u][nt].z, x[u][nt].w);
      }
    }
    // (5) every lane's operands have been consumed by the warp-wide MMAs: release the slot
    __syncwarp();
    if (lane == 0 && gi + kSlots < groups) mbar_arrive(empty(slot));
    // (6) scale and accumulate in increasing k; a row boundary finishes the segment
#pragma unroll
    for (int u = 0; u < kGroupTiles; ++u) {
      if (u < batch) {
        const bool is_w4 = (rec[u].offset_flag & kW4Flag) != 0;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          float s0, s1;
          if (p.scale_mode == AQ_SCALE_TOKEN) {
            s0 = __fmul_rn(token_scale[nt][0], rec[u].scale);
            s1 = __fmul_rn(token_scale[nt][1], rec[u].scale);
          } else {
            // tokens 8*nt .. 8*nt+7 share the scale of their 16-row group
            const float a_s = (nt * 8 < rows) ? p.act_scales[static_cast<int64_t>(nt >> 1) * n_k + kt] : 0.0f;
            s0 = s1 = __fmul_rn(a_s, rec[u].scale);
          }
          acc[nt][0] = __fadd_rn(acc[nt][0], __fmul_rn(static_cast<float>(d[u][nt][0]), s0));
          acc[nt][1] = __fadd_rn(acc[nt][1], __fmul_rn(static_cast<float>(d[u][nt][1]), s1));
          acc[nt][2] = __fadd_rn(acc[nt][2], __fmul_rn(static_cast<float>(d[u][nt][2]), s0));
          acc[nt][3] = __fadd_rn(acc[nt][3], __fmul_rn(static_cast<float>(d[u][nt][3]), s1));
          if (p.acc_dump != nullptr) {
            const int shift = is_w4 ? 4 : 0;
            const int tok = nt * 8 + 2 * c;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const int t = tok + (q & 1);
              const int col = n_a + ((q & 2) ? 8 : 0);
              if (t < rows) {
                p.acc_dump[((static_cast<int64_t>(t) * p.n_j + j) * n_k + kt) * kTile + col] = d[u][nt][q] >> shift;
              }
            }
          }
        }
        if (++kt == n_k) {
          flush(n_k);
          kt = 0;
          seg_k_lo = 0;
          ++j;
        }
      }
    }
  }
  if (kt != seg_k_lo && *abort_flag == 0) flush(kt);  // the range ended inside a row
}

int smem_bytes(int mt) {
  return kSlots * kSlotBytes + 8 * mt * kTile * 4 + kMaxRecords * 8 + kNumBars * 8 + 16;
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

int64_t partial_bytes(int ctas, int nt) { return 2LL * ctas * 8 * nt * kTile * 4; }

}  // namespace

int decode_ctas(int n_j, int n_k) {
  const int64_t total = static_cast<int64_t>(n_j) * n_k;
  const int64_t sms = num_sms();
  int64_t ctas = sms;
  while ((total + ctas - 1) / ctas > kMaxRecords) ctas += sms;
  return static_cast<int>(total < ctas ? total : ctas);
}

int64_t decode_workspace_bytes(int64_t m, int n_j, int n_k) {
  const int nt = m <= 8 ? 1 : (m <= 16 ? 2 : 4);
  return kCounterBytes + partial_bytes(decode_ctas(n_j, n_k), nt);
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
  return a.m <= 8 ? launch_mt<1>(p, stream) : (a.m <= 16 ? launch_mt<2>(p, stream) : launch_mt<4>(p, stream));
}

#ifdef AQ_TRACE
extern "C" __attribute__((visibility("default"))) int aq_debug_read_trace(long long* dst) {
  return static_cast<int>(cudaMemcpyFromSymbol(dst, g_trace, sizeof(long long) * 4096));
}
#endif

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
