// Persistent decode kernel: packed W4/W8 x A8 GEMV/GEMM for at most 16 rows.
//
// At decode sizes a whole layer is a few microseconds of HBM traffic, so the kernel
// is built to keep one uninterrupted byte stream per SM.  The layer's tiles are
// stored in (j, k) order in the prepared image; that 1-D sequence of T tiles is cut
// into G equal contiguous ranges, one per CTA, one CTA per SM ("stream-K").  A range
// is contiguous in memory, so the producer warp streams it through a shared-memory
// ring with ONE bulk asynchronous copy per slot of eight tiles (up to 32 KiB, counted
// on the slot's mbarrier).  The first ring fill is issued before the grid dependency
// is resolved, so under programmatic dependent launch it overlaps the preceding kernel.
//
// Sixteen consumer warps each take whole tiles (tile i of the range goes to warp
// i % 16), so sixteen tiles are in progress at once and every warp's waits, loads and
// MMAs overlap with the others'.  Inside a warp the weights are the 16-row MMA operand
// (mma.sync.m16n8k32.s8: 16 output columns) and up to eight activation rows
// ("tokens") the 8-column operand; activation vectors come straight from global
// memory (a few KiB, L1/L2 resident) and are requested one tile ahead.
//
// Summation order (all FP32, separately rounded multiply and add as in
// alignquant/kernels/cuda/linear.cu:956-963): a warp adds its tiles of a row segment
// in increasing k; the sixteen warp sums are added in warp order; the partial sums of
// the ranges that share a tile row are added in range order (the analogue of the
// reference's split-K reducer, linear.cu:1339-1343).  The order is fixed by the
// problem shape and the SM count, never by timing.
//
// A CTA range may start and end in the middle of a tile row.  A row that lies entirely
// inside one range is finished by that CTA.  Otherwise each CTA writes its partial
// FP32 tile to a workspace slot and bumps the row's counter; the CTA that arrives last
// sums the slots, applies the inverse output transform and stores the row.  Counters
// return to zero, so the workspace only has to be zeroed once by its owner.  Nothing
// spins on another CTA; every mbarrier wait is bounded (aq_ptx.cuh).
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
  float* partials;    // [2 * ctas][8 * NT][64]
  int32_t* counters;  // [n_j], zero between launches
  int64_t m;
  int64_t total_tiles;
  int n_j;
  int n_k;
  int ctas;
  int scale_mode;
  int out_dtype;
  // look-ahead prefetch of the next projection's image into L2 (prefetch_bytes == 0: none)
  const uint8_t* prefetch;
  int64_t prefetch_bytes;
};

constexpr int kGroupTiles = 8;  // tiles per ring slot: one copy and one full/empty barrier pair per slot
constexpr int kSlots = 4;       // ring depth in slots (32 tiles, 128 KiB)
constexpr int kSlotBytes = kGroupTiles * kW8TileBytes;
constexpr int kConsumerWarps = 16;
constexpr int kConsumerThreads = kConsumerWarps * 32;
constexpr int kThreads = kConsumerThreads + 32;
constexpr int kMaxRecords = 1024;
constexpr int kNumBars = 2 * kSlots;
constexpr int kMaxCounterRows = 16384;  // counters occupy a fixed region so that one workspace serves any layer
constexpr int64_t kCounterBytes = static_cast<int64_t>(kMaxCounterRows) * 4;

__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, 512;" ::: "memory"); }

// first tile of CTA i, and the CTA that owns tile t, for T tiles cut into G ranges
__device__ __forceinline__ int64_t range_begin(int64_t i, int64_t total, int ctas) { return i * total / ctas; }
__device__ __forceinline__ int owner_of(int64_t t, int64_t total, int ctas) {
  return static_cast<int>(((t + 1) * ctas - 1) / total);
}

// Lane (g, c) = (lane/4, lane%4) of a consumer warp holds, for column group q = 0..3,
// the weight vectors of columns 16q+g and 16q+g+8 and the activation vector of token
// 8*pass+g, all for k in [16c, 16c+16).  MMA results: d[0], d[1] = column 16q+g, tokens
// 8*pass+2c, +1; d[2], d[3] = column 16q+g+8, same tokens.
//
// Shared memory: [ring kSlots x 32 KiB][slabs 16 x (8*NT) x 64 f32][tile (8*NT) x 64 f32]
//                [records][barriers][flags]
template <int NT>
__global__ void __launch_bounds__(kThreads, 1) decode_linear_kernel(const DecodeParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  constexpr int kRows = 8 * NT;
  uint8_t* ring = smem;
  float* slabs = reinterpret_cast<float*>(smem + kSlots * kSlotBytes);
  float* tile = slabs + kConsumerWarps * kRows * kTile;
  TileRecord* recs = reinterpret_cast<TileRecord*>(tile + kRows * kTile);
  uint64_t* bars = reinterpret_cast<uint64_t*>(recs + kMaxRecords);
  volatile uint32_t* abort_flag = reinterpret_cast<uint32_t*>(bars + kNumBars);
  volatile uint32_t* last_flag = abort_flag + 1;
  volatile uint32_t* segment_abort = abort_flag + 2;  // the abort flag as thread 0 saw it between two barriers

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

  if (threadIdx.x == 0) {
    for (int s = 0; s < kSlots; ++s) {
      mbar_init(full(s), 1);
      mbar_init(empty(s), kGroupTiles);
    }
    *abort_flag = 0;
    mbar_init_fence();
    fence_proxy_async();
  }
  __syncthreads();

  const TileRecord* my_records = p.records + t0;
  const bool producer = warp == kConsumerWarps;

  // First ring fill: weights do not depend on the preceding kernel, so these copies are
  // issued before the grid dependency is resolved.  Lane l fetches slot l.
  if (producer && lane < kSlots && lane < groups) {
    const int first = lane * kGroupTiles;
    const int last = (first + kGroupTiles < count ? first + kGroupTiles : count) - 1;
    const TileRecord rf = my_records[first];
    const TileRecord rl = my_records[last];
    const uint32_t bytes = span_bytes(rf, rl);
    mbar_expect_tx(full(lane), bytes);
    bulk_copy(ring_addr + lane * kSlotBytes,
              p.payload + static_cast<int64_t>(rf.offset_flag & ~kW4Flag) * kW4TileBytes, bytes, full(lane));
  }
  // Look-ahead: the L2 cache fetches the image of the projection that runs next while this one
  // streams; requested after this CTA's own first fill.
  if (producer && lane == 0 && p.prefetch_bytes > 0) prefetch_slice_l2(p.prefetch, p.prefetch_bytes, blockIdx.x, gridDim.x);
  for (int i = threadIdx.x; i < count; i += kThreads) recs[i] = my_records[i];
  grid_launch_dependents();
  grid_dependency_wait();  // activations, scales, workspace and output belong to earlier kernels
  __syncthreads();

  if (producer) {
    // ---- refills: one copy per slot -----------------------------------------------------
    if (lane == 0) {
      for (int gi = kSlots; gi < groups; ++gi) {
        const int slot = gi % kSlots;
        if (!mbar_wait(empty(slot), ((gi / kSlots) - 1) & 1, abort_flag, &g_decode_status, 21)) break;
        const int first = gi * kGroupTiles;
        const int last = (first + kGroupTiles < count ? first + kGroupTiles : count) - 1;
        const TileRecord rf = recs[first];
        const uint32_t bytes = span_bytes(rf, recs[last]);
        mbar_expect_tx(full(slot), bytes);
        bulk_copy(ring_addr + slot * kSlotBytes,
                  p.payload + static_cast<int64_t>(rf.offset_flag & ~kW4Flag) * kW4TileBytes, bytes, full(slot));
      }
    }
    return;
  }

  // ---- consumers ------------------------------------------------------------------------
  const int g = lane >> 2;
  const int c = lane & 3;
  const int64_t k_bytes = static_cast<int64_t>(n_k) * kTile;
  // byte offsets of this lane's weight vector for column g of a 16-column group
  const uint32_t w8_off = static_cast<uint32_t>(g * 64 + ((c ^ ((g >> 1) & 3)) << 4));
  const uint32_t w4_off = static_cast<uint32_t>(g * 32 + (c >> 1) * 16);
  const int w4_shift = (c & 1) ? 0 : 4;
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

  auto load_x = [&](int i, uint4 (&x)[NT]) {
    const int kt = static_cast<int>((t0 + i) % n_k);
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      x[nt] = make_uint4(0, 0, 0, 0);
      if (nt * 8 + g < rows) x[nt] = ldg_x(x_lane[nt] + static_cast<int64_t>(kt) * kTile);
    }
  };

  float acc[NT][4][4];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
    for (int q = 0; q < 4; ++q) {
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[nt][q][e] = 0.0f;
    }
  }

  bool first_segment = true;
  int pos = 0;  // first tile (index inside the range) of the current row segment
  // this warp's next tile and its activation vectors, requested one tile ahead
  int mine = warp;
  uint4 x_next[NT];
  if (mine < count) load_x(mine, x_next);

  while (pos < count) {
    const int64_t t_first = t0 + pos;
    const int j = static_cast<int>(t_first / n_k);
    const int k_lo = static_cast<int>(t_first - static_cast<int64_t>(j) * n_k);
    const int64_t row_end = static_cast<int64_t>(j + 1) * n_k;
    const int seg_tiles = static_cast<int>((row_end < t1 ? row_end : t1) - t_first);
    const int seg_end = pos + seg_tiles;
    const bool whole_row = k_lo == 0 && seg_tiles == n_k;

    for (; mine < seg_end; mine += kConsumerWarps) {
      const int i = mine;
      const int gi = i / kGroupTiles;
      const int slot = gi % kSlots;
      const int kt = k_lo + (i - pos);
      uint4 x[NT];
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) x[nt] = x_next[nt];
      if (i + kConsumerWarps < count) load_x(i + kConsumerWarps, x_next);
      // A wait that gives up (or sees another thread's abort) only leaves the tile loop: the warp
      // still goes to the barriers below, where all sixteen warps leave together.
      if (!mbar_wait(full(slot), (gi / kSlots) & 1, abort_flag, &g_decode_status, 22)) break;
      const TileRecord rec = recs[i];
      const TileRecord rec0 = recs[gi * kGroupTiles];
      const bool is_w4 = (rec.offset_flag & kW4Flag) != 0;
      const uint8_t* staged = ring + slot * kSlotBytes +
                              ((rec.offset_flag & ~kW4Flag) - (rec0.offset_flag & ~kW4Flag)) * kW4TileBytes;
      int d[NT][4][4];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const uint8_t* group = staged + q * (is_w4 ? 16 * 32 : 16 * 64);
        const uint4 wa = weight_vector(group, is_w4, w8_off, w4_off, w4_shift);
        const uint4 wb = weight_vector(group + (is_w4 ? 8 * 32 : 8 * 64), is_w4, w8_off, w4_off, w4_shift);
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          d[nt][q][0] = d[nt][q][1] = d[nt][q][2] = d[nt][q][3] = 0;
          mma_s8(d[nt][q], wa.x, wb.x, wa.y, wb.y, x[nt].x, x[nt].y);
          mma_s8(d[nt][q], wa.z, wb.z, wa.w, wb.w, x[nt].z, x[nt].w);
        }
      }
      // every lane's operands have been consumed by the warp-wide MMAs: this tile is done
      __syncwarp();
      if (lane == 0 && gi + kSlots < groups) mbar_arrive(empty(slot));
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        float s0, s1;
        if (p.scale_mode == AQ_SCALE_TOKEN) {
          s0 = __fmul_rn(token_scale[nt][0], rec.scale);
          s1 = __fmul_rn(token_scale[nt][1], rec.scale);
        } else {
          // tokens 8*nt .. 8*nt+7 share the scale of their 16-row group
          const float a_s = (nt * 8 < rows) ? p.act_scales[static_cast<int64_t>(nt >> 1) * n_k + kt] : 0.0f;
          s0 = s1 = __fmul_rn(a_s, rec.scale);
        }
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          acc[nt][q][0] = __fadd_rn(acc[nt][q][0], __fmul_rn(static_cast<float>(d[nt][q][0]), s0));
          acc[nt][q][1] = __fadd_rn(acc[nt][q][1], __fmul_rn(static_cast<float>(d[nt][q][1]), s1));
          acc[nt][q][2] = __fadd_rn(acc[nt][q][2], __fmul_rn(static_cast<float>(d[nt][q][2]), s0));
          acc[nt][q][3] = __fadd_rn(acc[nt][q][3], __fmul_rn(static_cast<float>(d[nt][q][3]), s1));
        }
        if (p.acc_dump != nullptr) {
          const int shift = is_w4 ? 4 : 0;
          const int tok = nt * 8 + 2 * c;
#pragma unroll
          for (int q = 0; q < 4; ++q) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const int t = tok + (e & 1);
              const int col = q * 16 + g + ((e & 2) ? 8 : 0);
              if (t < rows) {
                p.acc_dump[((static_cast<int64_t>(t) * p.n_j + j) * n_k + kt) * kTile + col] = d[nt][q][e] >> shift;
              }
            }
          }
        }
      }
    }
    // ---- finish the segment: combine the sixteen warp sums in warp order --------------------
    {
      float* slab = slabs + warp * kRows * kTile;
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        const int tok = nt * 8 + 2 * c;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          slab[tok * kTile + q * 16 + g] = acc[nt][q][0];
          slab[(tok + 1) * kTile + q * 16 + g] = acc[nt][q][1];
          slab[tok * kTile + q * 16 + g + 8] = acc[nt][q][2];
          slab[(tok + 1) * kTile + q * 16 + g + 8] = acc[nt][q][3];
#pragma unroll
          for (int e = 0; e < 4; ++e) acc[nt][q][e] = 0.0f;
        }
      }
    }
    consumer_sync();
    // One thread samples the abort flag between the two barriers and every warp reads that sample
    // after the second one, so the decision to leave is the same in all sixteen warps whenever the
    // flag was raised (the producer may raise it at any time).
    if (threadIdx.x == 0) *segment_abort = *abort_flag;
    for (int e = threadIdx.x; e < kRows * kTile; e += kConsumerThreads) {
      float v = slabs[e];
#pragma unroll
      for (int w = 1; w < kConsumerWarps; ++w) v = __fadd_rn(v, slabs[w * kRows * kTile + e]);
      tile[e] = v;
    }
    consumer_sync();
    // Aborting: nothing of this segment is published, counted or stored.  The workspace
    // counters of rows already counted stay as they are (zero it again after AQ_ERR_DEVICE).
    if (*segment_abort != 0) break;
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
    consumer_sync();  // slabs, tile and the last-arriver flag are reused by the next segment
    first_segment = false;
    pos = seg_end;
  }
}

int smem_bytes(int mt) {
  return kSlots * kSlotBytes + (kConsumerWarps + 1) * 8 * mt * kTile * 4 + kMaxRecords * 8 + kNumBars * 8 + 16;  // 16: three flag words
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
  const int nt = m <= 8 ? 1 : 2;
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
  p.prefetch = static_cast<const uint8_t*>(a.prefetch);
  p.prefetch_bytes = a.prefetch != nullptr ? a.prefetch_bytes : 0;
  return a.m <= 8 ? launch_mt<1>(p, stream) : launch_mt<2>(p, stream);
}

// ---- allocation-free variant ------------------------------------------------------------
// Scratch for callers that cannot hand over a workspace (see aq_linear_decode_static in
// the header): arrival counters followed by partial tiles for up to kStaticMaxCtas
// ranges of 16 rows.  Lives in every device context that loads the library.
constexpr int kStaticMaxCtas = 256;
constexpr int64_t kStaticScratchBytes = kCounterBytes + 2LL * kStaticMaxCtas * 16 * kTile * 4;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

int64_t decode_static_scratch_bytes() { return kStaticScratchBytes; }

int launch_decode_linear_static(const LinearArgs& args, cudaStream_t stream) {
  // Everything that can be refused is refused first: no stream work and no symbol look-up on an
  // error path.
  if (args.n_j > kMaxCounterRows) {
    return fail(AQ_ERR_INVALID, "the decode kernel supports N up to %d, got %lld", kMaxCounterRows * kTile,
                static_cast<long long>(args.n_j) * kTile);
  }
  const int64_t need = decode_workspace_bytes(args.m, args.n_j, args.n_k);
  if (need > kStaticScratchBytes) {
    return fail(AQ_ERR_WORKSPACE,
                "this layer needs %lld bytes of scratch, the built-in scratch holds %lld; use aq_linear with a "
                "caller-owned workspace",
                static_cast<long long>(need), static_cast<long long>(kStaticScratchBytes));
  }
  // In host code `g_static_scratch` is only a handle for the symbol; the device address
  // has to be looked up, once per device, with that device current.
  static std::mutex mutex;
  static void* device_address[64] = {nullptr};
  int device = 0;
  int rc = check_cuda(cudaGetDevice(&device), "cudaGetDevice");
  if (rc != AQ_OK) return rc;
  if (device < 0 || device >= 64) return fail(AQ_ERR_INVALID, "device index %d is not supported", device);
  void* scratch = nullptr;
  {
    std::lock_guard<std::mutex> lock(mutex);
    if (device_address[device] == nullptr) {
      void* address = nullptr;
      rc = check_cuda(cudaGetSymbolAddress(&address, g_static_scratch), "cudaGetSymbolAddress(static scratch)");
      if (rc != AQ_OK) return rc;
      device_address[device] = address;
    }
    scratch = device_address[device];
  }
  // The array keeps whatever the previous call left behind; only the arrival counters of
  // the rows this call touches have to start at zero.
  rc = check_cuda(cudaMemsetAsync(scratch, 0, static_cast<size_t>(args.n_j) * sizeof(int32_t), stream),
                  "cudaMemsetAsync(static scratch counters)");
  if (rc != AQ_OK) return rc;
  LinearArgs a = args;
  a.workspace = scratch;
  a.workspace_bytes = kStaticScratchBytes;
  return launch_decode_linear(a, stream);
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
