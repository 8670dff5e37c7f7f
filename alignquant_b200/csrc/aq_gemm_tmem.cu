// Mixed W4/W8 x A8 GEMM for large row counts on the Blackwell tensor cores (sm_100a).
//
// One CTA computes a 128-row x 256-column output tile (four 64-column weight tile
// rows) and walks K in 64-wide steps through an 8-stage shared-memory ring.  Roles of the
// sixteen warps of that layout (the 128-column layouts are described at struct Layout):
//   * warps 6-7 stream the weights: one bulk asynchronous copy (cp.async.bulk) per tile
//     of the prepared image and K step.  A W8 tile is stored in the K-major 64-byte-swizzle
//     operand layout, so its copy signals the stage's "ready" mbarrier directly; a W4 tile
//     lands packed in the first half of its operand slot.  Issuing a bulk copy costs its
//     warp about 150 cycles whatever its size, which is why the copies of a step are spread
//     over several warps;
//   * warps 0-3, one per weight tile row of the CTA tile, widen landed W4 tiles in place
//     (value 16*w: one shift, one mask), publish them to the asynchronous proxy and arrive
//     on "ready";
//   * warp 5 streams the activations: one tensor-map copy (cp.async.bulk.tensor.2d,
//     64-byte swizzle) per K step brings the 128 x 64 int8 block of the row-major
//     activation matrix into the same operand layout; rows past M read as zero;
//   * warp 4: one thread issues tcgen05.mma kind::i8 (M=128, N<=256, K=32, twice per
//     step) into one of two 256-column tensor-memory accumulators and commits to
//     mbarriers (stage free, accumulator full);
//   * warps 8-15 drain: tcgen05.ld the int32 accumulator, convert, and add
//     float(int32) * (activation scale * tile scale) into FP32 registers -- integer
//     accumulation never spans two K64 tiles because every tile has its own scale
//     (alignquant/kernels/cuda/linear.cu:951-963).  By default a tile is added with one
//     packed fused multiply-add; the reference kernels' separately rounded multiply and add
//     is a library option (AQ_OPT_GEMM_ROUNDING).
// The epilogue stages rows through shared memory so that global stores are coalesced
// and applies the inverse output transform (linear.cu:983-1040) where a tile has one.
//
// Every mbarrier wait is bounded; on a time-out the CTA raises a device status word
// (read by aq_device_status), stops issuing, gives copies in flight time to land,
// frees its tensor memory and returns.
#include <cooperative_groups.h>
#include <cuda.h>

#include <mutex>

#include "aq_common.cuh"
#include "aq_ptx.cuh"
#include "aq_tile_math.cuh"
#include "aq_tcgen05.cuh"

namespace cg = cooperative_groups;

namespace aq {

__device__ int g_gemm_status = 0;

namespace {

constexpr int kBM = 128;
constexpr int kABytes = kBM * kTile;  // 8192
constexpr int kMaxNk = 512;
constexpr int kEpiRowFloats = 65;

// Geometry and warp roles of a kernel variant.  TN = weight tile rows (64 columns each) of the
// CTA tile; kPaired = two small CTAs per SM instead of one large one.
//   large CTA (512 threads, one per SM): warps 0..TN-1 widen, 4 issues the MMAs, 5 streams the
//     activations, 6-7 the weights, 8-15 drain (lane quarter x column half); 512 tensor-memory
//     columns = 512 / (64 TN) accumulators.  With TN = 2 (four accumulators) warps 2-5 issue the
//     MMAs in turn and warp 6 also streams the activations.
//   paired CTA (256 threads, TN = 2, two per SM): warp 0 issues the MMAs, warp 1 streams
//     activations and weights, warps 2-3 widen, warps 4-7 drain (one per lane quarter, all 128
//     columns); 256 tensor-memory columns = two accumulators; six stages of 16 KiB.  The step
//     of one CTA (wait, load, convert, hand the accumulator back) is a chain of latencies; the
//     second CTA of the SM fills the gaps of the first.
template <int TN, bool kPaired>
struct Layout {
  static_assert(!kPaired || TN == 2, "the paired layout is 128 columns wide");
  static constexpr int kThreads = kPaired ? 256 : 512;
  static constexpr int kCtasPerSm = kPaired ? 2 : 1;
  static constexpr int kStages = kPaired ? 6 : 8;
  static constexpr int kTmemColumns = kPaired ? 256 : 512;
  static constexpr bool kNarrow = !kPaired && TN == 2;
  // MMA-issuing warps: warp kMmaWarp + i issues the K steps kt with kt % kMmaWarps == i.  Waiting
  // for operands and an accumulator, two MMAs and two commits cost the issuing warp several
  // hundred cycles per step; with four 128-column accumulators that, not the tensor pipe or the
  // drain, bounds a step, so the one-CTA 128-column layout spreads the steps over four warps.
  static constexpr int kMmaWarp = kPaired ? 0 : kNarrow ? 2 : 4;
  static constexpr int kMmaWarps = kNarrow ? 4 : 1;
  static constexpr int kActWarp = kPaired ? 1 : kNarrow ? 6 : 5;
  static constexpr int kFirstCopyWarp = kPaired ? 1 : 6;
  static constexpr int kCopyWarps = kPaired ? 1 : 2;
  static constexpr int kFirstWidenWarp = kPaired ? 2 : 0;
  static constexpr int kFirstDrainWarp = kPaired ? 4 : 8;
  static constexpr int kDrainWarps = kPaired ? 4 : 8;
  static constexpr int kIdleRegs = 40;
  static constexpr int kDrainRegs = 216;
  static constexpr int kCols = TN * kTile;
  static constexpr int kBBytes = TN * kW8TileBytes;
  static constexpr int kStageBytes = kABytes + kBBytes;  // a multiple of the 1024-byte operand alignment
  static constexpr int kRecBytes = TN * kMaxNk * static_cast<int>(sizeof(TileRecord));
  static constexpr int kAccs = kTmemColumns / kCols;
  // ready[S], empty[S], packed[S][TN], acc_full[kAccs], acc_empty[kAccs], final[kMmaWarps]
  static constexpr int kNumBars = (2 + TN) * kStages + 2 * kAccs + kMmaWarps;
  static constexpr int kSmemBytes = kStages * kStageBytes + kRecBytes + kNumBars * 8 + 16;
  static constexpr int kHalves = kDrainWarps / 4;        // column groups of the drain warps
  static constexpr int kTilesPerHalf = TN / kHalves;     // weight tile rows drained by one warp
  static constexpr int kChunks = 4 * kTilesPerHalf;      // 16-column chunks per drain warp and K step
  static constexpr int kTilesPerCopyWarp = TN / kCopyWarps;
  static_assert(kBM * (kCols + 1) * 4 <= kStages * kStageBytes, "the split-K exchange tile must fit into the ring");
  static_assert(kDrainWarps * 32 * kEpiRowFloats * 4 <= kStages * kStageBytes, "the epilogue rows must fit into the ring");
};

struct GemmParams {
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

// acc[16*c .. 16*c+15] += float(v) * scale, multiply and add rounded separately (operation
// order of linear.cu:958-962); the two sums of a pair are added with one packed instruction
template <int NACC>
__device__ __forceinline__ void drain_chunk(uint64_t (&acc)[NACC], int c, const int (&v)[16], float scale) {
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const float p0 = __fmul_rn(__int2float_rn(v[2 * i]), scale);
    const float p1 = __fmul_rn(__int2float_rn(v[2 * i + 1]), scale);
    acc[c * 8 + i] = add2(acc[c * 8 + i], pack2(__float_as_uint(p0), __float_as_uint(p1)));
  }
}

// acc[16*c .. 16*c+15] = fma(float(v), scale, acc): one rounding per tile, two sums per
// instruction (fma.rn.f32x2).
template <int NACC>
__device__ __forceinline__ void drain_chunk_fused(uint64_t (&acc)[NACC], int c, const int (&v)[16], uint64_t scale2) {
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const uint64_t f = pack2(__float_as_uint(__int2float_rn(v[2 * i])), __float_as_uint(__int2float_rn(v[2 * i + 1])));
    acc[c * 8 + i] = fma2(f, scale2, acc[c * 8 + i]);
  }
}

// 64 consecutive FP32 sums (32 packed pairs) of one row -> out[first .. first + 63] with 16-byte stores.
__device__ __forceinline__ void store_row64(void* out, int dtype, int64_t first, const uint64_t* acc) {
  if (dtype == AQ_F32) {
    float4* dst = reinterpret_cast<float4*>(static_cast<float*>(out) + first);
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      float a, b, c, d;
      unpack2(acc[2 * i], a, b);
      unpack2(acc[2 * i + 1], c, d);
      dst[i] = make_float4(a, b, c, d);
    }
  } else {
    uint4* dst = reinterpret_cast<uint4*>(static_cast<uint16_t*>(out) + first);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      uint32_t w[4];
#pragma unroll
      for (int h = 0; h < 4; ++h) {
        float a, b;
        unpack2(acc[4 * i + h], a, b);
        if (dtype == AQ_BF16) {
          const __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
          w[h] = *reinterpret_cast<const uint32_t*>(&v);
        } else {
          const __half2 v = __floats2half2_rn(a, b);
          w[h] = *reinterpret_cast<const uint32_t*>(&v);
        }
      }
      dst[i] = make_uint4(w[0], w[1], w[2], w[3]);
    }
  }
}

// Debug aid: the exact integer tile sums (W4 tiles were fed 16*w to the MMA).
__device__ __forceinline__ void dump_chunk(int32_t* tile_dump, int first_col, const int (&v)[16], const TileRecord& r) {
  if (tile_dump == nullptr) return;
  const int shift = (r.offset_flag & kW4Flag) ? 4 : 0;
  int4* o = reinterpret_cast<int4*>(tile_dump + first_col);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    o[i] = make_int4(v[4 * i] >> shift, v[4 * i + 1] >> shift, v[4 * i + 2] >> shift, v[4 * i + 3] >> shift);
  }
}

template <int TN, bool kPaired, bool kDump, bool kFused>
__global__ void __launch_bounds__(Layout<TN, kPaired>::kThreads, Layout<TN, kPaired>::kCtasPerSm)
tmem_gemm_kernel(const __grid_constant__ CUtensorMap x_map, const GemmParams p) {
  using S = Layout<TN, kPaired>;
  constexpr int kStages = S::kStages;
  constexpr int kStageBytes = S::kStageBytes;
  constexpr int kAccs = S::kAccs;
  constexpr int kTilesN = TN;
  constexpr int kThreads = S::kThreads;
  constexpr int kDrainWarps = S::kDrainWarps;
  constexpr int kFirstDrainWarp = S::kFirstDrainWarp;
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* stages = smem;
  TileRecord* rec_smem = reinterpret_cast<TileRecord*>(smem + kStages * kStageBytes);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kStages * kStageBytes + S::kRecBytes);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + S::kNumBars);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int n_k = p.n_k;
  // split-K over a thread-block cluster along z: this CTA walks K steps [k_begin, k_begin + steps)
  cg::cluster_group cluster = cg::this_cluster();
  const int split_k = static_cast<int>(cluster.num_blocks());
  const int split = static_cast<int>(cluster.block_rank());
  const int k_begin = static_cast<int>(static_cast<int64_t>(n_k) * split / split_k);
  const int steps = static_cast<int>(static_cast<int64_t>(n_k) * (split + 1) / split_k) - k_begin;
  const int j0 = blockIdx.x * kTilesN;
  const int tiles_here = min(kTilesN, p.n_j - j0);
  const int64_t m0 = static_cast<int64_t>(blockIdx.y) * kBM;

  const uint32_t bar0 = smem_u32(bars);
  auto ready = [&](int s) { return bar0 + 8u * s; };
  auto empty = [&](int s) { return bar0 + 8u * (kStages + s); };
  auto packed = [&](int s, int t) { return bar0 + 8u * (2 * kStages + TN * s + t); };
  auto acc_full = [&](int b) { return bar0 + 8u * ((2 + TN) * kStages + b); };
  auto acc_empty = [&](int b) { return bar0 + 8u * ((2 + TN) * kStages + kAccs + b); };
  auto final_bar = [&](int i) { return bar0 + 8u * ((2 + TN) * kStages + 2 * kAccs + i); };

  // one thread per barrier: the initialisations would otherwise run one after the other
  if (threadIdx.x < S::kNumBars) {
    const int i = threadIdx.x;
    uint32_t count = 1;  // empty, packed, acc_full and final: one arrival (a commit or a copy's expect_tx)
    if (i < kStages) {
      count = static_cast<uint32_t>(tiles_here) + 1;  // ready: one arrival per weight stream + activations
    } else if (i >= (2 + TN) * kStages + kAccs && i < (2 + TN) * kStages + 2 * kAccs) {
      count = kDrainWarps;  // acc_empty: one arrival per drain warp
    }
    mbar_init(bar0 + 8u * i, count);
    if (i == 0) *abort_flag = 0;
    mbar_init_fence();
    fence_proxy_async();
  }
  for (int i = threadIdx.x; i < tiles_here * steps; i += kThreads) {
    const int t = i / steps, kt = i % steps;  // kt counts from k_begin everywhere below
    rec_smem[t * kMaxNk + kt] = p.records[static_cast<int64_t>(j0 + t) * n_k + k_begin + kt];
  }
  if (warp == S::kMmaWarp) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(tmem_slot)),
                 "r"(static_cast<uint32_t>(S::kTmemColumns))
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp < kFirstDrainWarp) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(S::kIdleRegs));
    // the warp that streams the activations may also stream weight tiles (paired layout)
    const bool copies_weights = warp >= S::kFirstCopyWarp && warp < S::kFirstCopyWarp + S::kCopyWarps;
    const bool copies_acts = warp == S::kActWarp;
    if (warp >= S::kFirstWidenWarp && warp < S::kFirstWidenWarp + tiles_here) {
      // ---------------- W4 widening of tile row j0 + t -----------------------------------
      // W8 tiles need no work here: their copy completes "ready" by itself.
      const int t = warp - S::kFirstWidenWarp;
      const TileRecord* recs = rec_smem + t * kMaxNk;
      uint32_t packed_parity = 0;  // bit s: phase the next wait on packed(s, t) looks for
      for (int kt = 0; kt < steps; ++kt) {
        if ((recs[kt].offset_flag & kW4Flag) == 0) continue;
        const int s = kt % kStages;
        int landed = 1;
        if (lane == 0) landed = mbar_wait(packed(s, t), (packed_parity >> s) & 1u, abort_flag, &g_gemm_status, 6) ? 1 : 0;
        if (__shfl_sync(0xffffffffu, landed, 0) == 0) break;
        packed_parity ^= 1u << s;
        // Widen in place.  Packed chunk q = 2*n + h (16 bytes) holds the k16 blocks 2h (low
        // nibbles) and 2h+1 (high nibbles) of row n; the widened row n takes bytes 64n..64n+63
        // of the slot, so every lane reads its four chunks before any lane writes.
        uint8_t* tile = stages + s * kStageBytes + kABytes + t * kW8TileBytes;
        uint4 pk[4];
#pragma unroll
        for (int r = 0; r < 4; ++r) pk[r] = *reinterpret_cast<const uint4*>(tile + (r * 32 + lane) * 16);
        __syncwarp();
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          const int q = r * 32 + lane;
          const int n = q >> 1, h = q & 1;
          uint4 lo, hi;
          lo.x = (pk[r].x << 4) & 0xf0f0f0f0u;
          lo.y = (pk[r].y << 4) & 0xf0f0f0f0u;
          lo.z = (pk[r].z << 4) & 0xf0f0f0f0u;
          lo.w = (pk[r].w << 4) & 0xf0f0f0f0u;
          hi.x = pk[r].x & 0xf0f0f0f0u;
          hi.y = pk[r].y & 0xf0f0f0f0u;
          hi.z = pk[r].z & 0xf0f0f0f0u;
          hi.w = pk[r].w & 0xf0f0f0f0u;
          uint8_t* row = tile + n * 64;
          const int swz = (n >> 1) & 3;
          *reinterpret_cast<uint4*>(row + (((2 * h) ^ swz) << 4)) = lo;
          *reinterpret_cast<uint4*>(row + (((2 * h + 1) ^ swz) << 4)) = hi;
        }
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) mbar_arrive(ready(s));
      }
    } else if (copies_weights || copies_acts) {
      // ---------------- operand copies ------------------------------------------------------
      // Issuing a bulk copy takes its warp about 150 cycles whatever the size, so in the large
      // layout the copies of a K step are spread over three warps (activations, two weight
      // streams) and kept apart from the widening.  Activations: one tensor-map copy per step
      // brings the 128 x 64 int8 block into the operand layout; rows past M read as zero.
      if (lane == 0) {
        const int t_first = copies_weights ? (warp - S::kFirstCopyWarp) * S::kTilesPerCopyWarp : 0;
        const int wait_code = copies_acts ? 3 : 1;
        for (int kt = 0; kt < steps; ++kt) {
          const int s = kt % kStages;
          if (kt >= kStages && !mbar_wait(empty(s), ((kt / kStages) - 1) & 1, abort_flag, &g_gemm_status, wait_code)) break;
          if (copies_acts) {
            mbar_expect_tx(ready(s), kABytes);
            tensor_copy_2d(smem_u32(stages + s * kStageBytes), &x_map, (k_begin + kt) * kTile, static_cast<int>(m0), ready(s));
          }
          if (copies_weights) {
#pragma unroll
            for (int i = 0; i < S::kTilesPerCopyWarp; ++i) {
              const int t = t_first + i;
              if (t >= tiles_here) break;
              const uint32_t of = rec_smem[t * kMaxNk + kt].offset_flag;
              const uint8_t* src = p.payload + static_cast<int64_t>(of & ~kW4Flag) * kW4TileBytes;
              const uint32_t dst = smem_u32(stages + s * kStageBytes + kABytes + t * kW8TileBytes);
              if (of & kW4Flag) {
                mbar_expect_tx(packed(s, t), kW4TileBytes);
                bulk_copy(dst, src, kW4TileBytes, packed(s, t));
              } else {
                mbar_expect_tx(ready(s), kW8TileBytes);
                bulk_copy(dst, src, kW8TileBytes, ready(s));
              }
            }
          }
        }
      }
      __syncwarp();
    } else if (warp >= S::kMmaWarp && warp < S::kMmaWarp + S::kMmaWarps) {
      // ---------------- MMA issuer(s) ------------------------------------------------
      // The whole warp walks the loop so that addresses and descriptors stay warp-uniform
      // values (the MMA takes them from uniform registers); one elected lane issues.  Steps
      // issued by different warps use different stages and different accumulators.
      const uint32_t idesc = instr_desc_i8(64 * tiles_here);
      const uint32_t stage0 = smem_u32(stages);
      const int issuer = warp - S::kMmaWarp;
      bool ok = true;
      for (int kt = issuer; kt < steps; kt += S::kMmaWarps) {
        const int s = kt % kStages;
        const int b = kt % kAccs;
        ok = warp_wait(ready(s), (kt / kStages) & 1, lane, abort_flag, &g_gemm_status, 2);
        ok = ok && warp_wait(acc_empty(b), (kt / kAccs) & 1, lane, abort_flag, &g_gemm_status, 5);
        if (!ok) break;
        tc_fence_after();
        const uint32_t a_addr = stage0 + static_cast<uint32_t>(s) * kStageBytes;
        const uint32_t b_addr = a_addr + kABytes;
        const uint32_t d = tmem_base + static_cast<uint32_t>(b * S::kCols);
        if (elect_one()) {
          // Both operands: rows of 64 bytes, the second K32 half of a row starts 32 bytes in.
          // Every K step starts a fresh integer sum: the first MMA overwrites the accumulator.
          tc_mma_i8(d, smem_desc_sw64(a_addr), smem_desc_sw64(b_addr), idesc, 0u);
          tc_mma_i8(d, smem_desc_sw64(a_addr + 32), smem_desc_sw64(b_addr + 32), idesc, 1u);
          tc_commit(empty(s));
          tc_commit(acc_full(b));
        }
        __syncwarp();
      }
      if (!ok && lane == 0) {
        // make sure nothing issued is still running before tensor memory is freed
        tc_commit(final_bar(issuer));
        for (uint32_t i = 0; i < (1u << 20) && !mbar_try_wait(final_bar(issuer), 0); ++i) {
        }
      }
      __syncwarp();
    }
    if (*abort_flag != 0) {
      // bulk copies may still be in flight: give them a bounded time to land before the CTA
      // and its shared memory go away
      for (int i = 0; i < 64; ++i) __nanosleep(2000);
    }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(S::kDrainRegs));
    // ---------------- drain: int32 accumulator -> scaled FP32 registers -------------
    const int quarter = warp & 3;       // tensor-memory lane quarter this warp may read
    constexpr int kTH = S::kTilesPerHalf;
    constexpr int kChunks = S::kChunks;
    const int half = (warp - kFirstDrainWarp) >> 2;  // column group: weight tile rows kTH*half ...
    const int row = quarter * 32 + lane;
    const int64_t grow = m0 + row;
    const bool row_valid = grow < p.m;
    const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                           static_cast<uint32_t>(half * kTH * kTile);
    uint64_t acc[32 * kTH];  // 64 * kTH FP32 sums as packed pairs
#pragma unroll
    for (int i = 0; i < 32 * kTH; ++i) acc[i] = 0ull;
    const float token_scale =
        (p.scale_mode == AQ_SCALE_TOKEN && row_valid) ? p.act_scales[grow] : 0.0f;
    const float* tile_scales =
        (p.scale_mode == AQ_SCALE_TILE && row_valid) ? p.act_scales + (grow >> 4) * n_k : nullptr;
    const TileRecord* recs = rec_smem + (kTH * half) * kMaxNk;

    tc_fence_before();
    __syncwarp();
    if (lane == 0) {  // every accumulator starts out free
      for (int b = 0; b < kAccs; ++b) mbar_arrive(acc_empty(b));
    }
    bool ok = true;
    if constexpr (kTH == 1) {
      // One weight tile (64 columns) per warp and K step: the whole slice of the accumulator is
      // loaded at once and the accumulator handed back BEFORE the arithmetic, so that it is held
      // only for the time of the loads.  What bounds a K step otherwise is not arithmetic but the
      // round trip of an accumulator (hand back, wake the MMA warp, MMA, commit, wake the drain
      // warps) divided by the number of accumulators the 512 tensor-memory columns hold.
      int v0[16], v1[16], v2[16], v3[16];
      for (int kt = 0; kt < steps; ++kt) {
        const int b = kt % kAccs;
        ok = warp_wait(acc_full(b), (kt / kAccs) & 1, lane, abort_flag, &g_gemm_status, 7);
        if (!ok) break;
        tc_fence_after();
        const uint32_t col = taddr + static_cast<uint32_t>(b * S::kCols);
        tc_ld16(col, v0);
        tc_ld16(col + 16, v1);
        tc_ld16(col + 32, v2);
        tc_ld16(col + 48, v3);
        tc_wait_ld(v0);
        tc_wait_ld(v1);
        tc_wait_ld(v2);
        tc_wait_ld(v3);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(acc_empty(b));
        const float a_scale = tile_scales != nullptr ? tile_scales[k_begin + kt] : token_scale;
        const TileRecord rec = recs[kt];
        const float scale = __fmul_rn(a_scale, rec.scale);
        const uint64_t scale2 = pack2(__float_as_uint(scale), __float_as_uint(scale));
        if (kFused) {
          drain_chunk_fused(acc, 0, v0, scale2);
          drain_chunk_fused(acc, 1, v1, scale2);
          drain_chunk_fused(acc, 2, v2, scale2);
          drain_chunk_fused(acc, 3, v3, scale2);
        } else {
          drain_chunk(acc, 0, v0, scale);
          drain_chunk(acc, 1, v1, scale);
          drain_chunk(acc, 2, v2, scale);
          drain_chunk(acc, 3, v3, scale);
        }
        if (kDump && row_valid && half < tiles_here) {
          int32_t* dump = p.acc_dump + ((grow * p.n_j + (j0 + half)) * n_k + k_begin + kt) * kTile;
          dump_chunk(dump, 0, v0, rec);
          dump_chunk(dump, 16, v1, rec);
          dump_chunk(dump, 32, v2, rec);
          dump_chunk(dump, 48, v3, rec);
        }
      }
    } else {
    // Software pipeline over 16-column chunks (four per weight tile) with two register
    // buffers: while the arithmetic of one chunk runs, the tensor-memory load of the next one
    // is in flight.  The accumulator goes back to the MMA thread as soon as its last chunk
    // has been loaded, before that chunk's arithmetic.
    int va[16], vb[16];
    ok = warp_wait(acc_full(0), 0, lane, abort_flag, &g_gemm_status, 7);
    if (ok) {
      tc_fence_after();
      tc_ld16(taddr, va);
    }
    for (int kt = 0; kt < steps && ok; ++kt) {
      const int b = kt % kAccs;
      const int b_next = (kt + 1) % kAccs;
      const uint32_t col = taddr + static_cast<uint32_t>(b * S::kCols);
      const float a_scale = tile_scales != nullptr ? tile_scales[k_begin + kt] : token_scale;
      TileRecord rec[kTH];
      float scale[kTH];
      uint64_t scale2[kTH];
      int32_t* dump[kTH];
#pragma unroll
      for (int t = 0; t < kTH; ++t) {
        rec[t] = recs[t * kMaxNk + kt];
        scale[t] = __fmul_rn(a_scale, rec[t].scale);
        scale2[t] = pack2(__float_as_uint(scale[t]), __float_as_uint(scale[t]));
        dump[t] = nullptr;
        if (kDump && row_valid && kTH * half + t < tiles_here) {
          dump[t] = p.acc_dump + ((grow * p.n_j + (j0 + kTH * half + t)) * n_k + k_begin + kt) * kTile;
        }
      }
#pragma unroll
      for (int c = 0; c < kChunks; ++c) {
        int (&cur)[16] = (c & 1) ? vb : va;
        int (&next)[16] = (c & 1) ? va : vb;
        tc_wait_ld(cur);
        if (c + 1 < kChunks) {
          tc_ld16(col + (c + 1) * 16, next);
        } else {
          // The last chunk has been loaded: this accumulator has been read completely.  The
          // next one is waited for before this one is handed back: a poll made after the
          // hand-over would queue behind the MMA thread, which starts issuing at that moment.
          // There is no dead-lock: the MMA of step kt+1 never needs the accumulator of step kt.
          if (kt + 1 < steps) ok = warp_wait(acc_full(b_next), ((kt + 1) / kAccs) & 1, lane, abort_flag, &g_gemm_status, 7);
          if (kt + 1 < steps && ok) {
            tc_fence_after();
            tc_ld16(taddr + static_cast<uint32_t>(b_next * S::kCols), next);
          }
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(acc_empty(b));
        }
        if (kFused) {
          drain_chunk_fused(acc, c, cur, scale2[c >> 2]);
        } else {
          drain_chunk(acc, c, cur, scale[c >> 2]);
        }
        if (kDump) dump_chunk(dump[c >> 2], (c & 3) * 16, cur, rec[c >> 2]);
      }
    }
    }

    // ---------------- epilogue: rows through shared memory, coalesced stores --------
    if (split_k > 1) {
      // split-K: the CTA's FP32 tile goes to shared memory (over the stage ring, rows padded by
      // one float so that a warp writing one row per lane hits 32 banks) for the exchange below
      float* xchg = reinterpret_cast<float*>(stages);
#pragma unroll
      for (int t = 0; t < kTH; ++t) {
#pragma unroll
        for (int c = 0; c < 32; ++c) {
          float lo, hi;
          unpack2(acc[t * 32 + c], lo, hi);
          float* dst = xchg + row * (S::kCols + 1) + (kTH * half + t) * kTile + 2 * c;
          dst[0] = lo;
          dst[1] = hi;
        }
      }
    } else if (ok) {
      float* region = reinterpret_cast<float*>(stages) + (warp - kFirstDrainWarp) * (32 * kEpiRowFloats);
      const int64_t n_cols = static_cast<int64_t>(p.n_j) * kTile;
#pragma unroll
      for (int t = 0; t < kTH; ++t) {
        const int tl = kTH * half + t;
        if (tl < tiles_here) {
          const int j = j0 + tl;
          const int32_t* row_meta = p.u_metadata ? p.u_metadata + static_cast<int64_t>(j) * 4 * kTile : nullptr;
          if (row_meta == nullptr || row_meta[0] == 0) {
            // No output transform: a thread owns 64 consecutive columns of its row, i.e. whole
            // 128-byte lines of the result, and stores them straight from its registers.
            if (row_valid) store_row64(p.out, p.out_dtype, grow * n_cols + static_cast<int64_t>(j) * kTile, &acc[t * 32]);
            continue;
          }
#pragma unroll
          for (int c = 0; c < 32; ++c) {
            float lo, hi;
            unpack2(acc[t * 32 + c], lo, hi);
            region[lane * kEpiRowFloats + 2 * c] = lo;
            region[lane * kEpiRowFloats + 2 * c + 1] = hi;
          }
          __syncwarp();
          const int32_t* meta =
              p.u_metadata ? p.u_metadata + static_cast<int64_t>(j) * 4 * kTile : nullptr;
          const bool has_u = meta != nullptr && meta[0] != 0;
          for (int r = 0; r < 32; ++r) {
            const int64_t gr = m0 + quarter * 32 + r;
            if (gr >= p.m) break;
            float lo = region[r * kEpiRowFloats + lane];
            float hi = region[r * kEpiRowFloats + lane + 32];
            if (has_u) inverse_u_row(lo, hi, meta, lane);
            const int64_t o = gr * n_cols + static_cast<int64_t>(j) * kTile + lane;
            store_any(p.out, p.out_dtype, o, lo);
            store_any(p.out, p.out_dtype, o + 32, hi);
          }
          __syncwarp();
        }
      }
    }
  }

  if (split_k > 1) {
    // ---------------- split-K exchange through cluster shared memory ------------------------
    // CTA r of the cluster finishes rows r, r + split_k, ...: it adds the split sums in split
    // order (the reference reducer's order, linear.cu:1339-1343), applies the inverse output
    // transform and stores.  The second barrier keeps every CTA's tile alive until read.
    cluster.sync();
    if (warp >= kFirstDrainWarp) {
      const float* xchg = reinterpret_cast<const float*>(stages);
      const int64_t n_cols = static_cast<int64_t>(p.n_j) * kTile;
      const float* remote[8];
#pragma unroll
      for (int s = 0; s < 8; ++s) remote[s] = cluster.map_shared_rank(xchg, s < split_k ? s : 0);
      const int64_t rows_left = p.m - m0 - split;  // owned rows: split, split + split_k, ... below p.m
      const int owned = rows_left <= 0 ? 0
                        : static_cast<int>(((rows_left < kBM - split ? rows_left : kBM - split) + split_k - 1) / split_k);
      const int pairs = owned * tiles_here;  // (row, weight tile row) pairs, dealt to the drain warps
      for (int q = warp - kFirstDrainWarp; q < pairs; q += kDrainWarps) {
        const int row = split + split_k * (q / tiles_here);
        const int tl = q % tiles_here;
        const int offset = row * (S::kCols + 1) + tl * kTile + lane;
        // all remote loads of the pair are issued before the first add
        float a[8], b[8];
#pragma unroll
        for (int s = 0; s < 8; ++s) {
          a[s] = 0.0f;
          b[s] = 0.0f;
          if (s < split_k) {
            a[s] = remote[s][offset];
            b[s] = remote[s][offset + 32];
          }
        }
        float lo = a[0], hi = b[0];
#pragma unroll
        for (int s = 1; s < 8; ++s) {
          if (s < split_k) {
            lo = __fadd_rn(lo, a[s]);
            hi = __fadd_rn(hi, b[s]);
          }
        }
        const int j = j0 + tl;
        const int32_t* meta = p.u_metadata ? p.u_metadata + static_cast<int64_t>(j) * 4 * kTile : nullptr;
        if (meta != nullptr && meta[0] != 0) inverse_u_row(lo, hi, meta, lane);
        const int64_t o = (m0 + row) * n_cols + static_cast<int64_t>(j) * kTile + lane;
        store_any(p.out, p.out_dtype, o, lo);
        store_any(p.out, p.out_dtype, o + 32, hi);
      }
    }
    cluster.sync();
  }

  tc_fence_before();
  __syncthreads();
  if (warp == S::kMmaWarp) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"(static_cast<uint32_t>(S::kTmemColumns))
                 : "memory");
  }
}

template <int TN, bool kPaired>
int launch_shape(const CUtensorMap& x_map, const GemmParams& p, bool dump, bool fused, int split, int device,
                 cudaStream_t stream) {
  using S = Layout<TN, kPaired>;
  static std::once_flag once[64];
  cudaError_t attr_status = cudaSuccess;
  std::call_once(once[device & 63], [&] {
    const void* kernels[4] = {
        reinterpret_cast<const void*>(tmem_gemm_kernel<TN, kPaired, false, false>),
        reinterpret_cast<const void*>(tmem_gemm_kernel<TN, kPaired, false, true>),
        reinterpret_cast<const void*>(tmem_gemm_kernel<TN, kPaired, true, false>),
        reinterpret_cast<const void*>(tmem_gemm_kernel<TN, kPaired, true, true>)};
    for (const void* kernel : kernels) {
      if (attr_status == cudaSuccess) {
        attr_status = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kSmemBytes);
      }
    }
  });
  int rc = check_cuda(attr_status, "cudaFuncSetAttribute(tmem_gemm_kernel)");
  if (rc != AQ_OK) return rc;
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(static_cast<unsigned>((p.n_j + TN - 1) / TN), static_cast<unsigned>((p.m + kBM - 1) / kBM),
                        static_cast<unsigned>(split));
  config.blockDim = dim3(S::kThreads, 1, 1);
  config.dynamicSmemBytes = static_cast<size_t>(S::kSmemBytes);
  config.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = static_cast<unsigned>(split);
  config.attrs = attr;
  config.numAttrs = 1;
  cudaError_t status;
  if (dump) {
    status = fused ? cudaLaunchKernelEx(&config, tmem_gemm_kernel<TN, kPaired, true, true>, x_map, p)
                   : cudaLaunchKernelEx(&config, tmem_gemm_kernel<TN, kPaired, true, false>, x_map, p);
  } else {
    status = fused ? cudaLaunchKernelEx(&config, tmem_gemm_kernel<TN, kPaired, false, true>, x_map, p)
                   : cudaLaunchKernelEx(&config, tmem_gemm_kernel<TN, kPaired, false, false>, x_map, p);
  }
  return check_cuda(status, "tensor-memory GEMM launch");
}

int device_sm_count(int* count) {
  int device = 0;
  int rc = check_cuda(cudaGetDevice(&device), "cudaGetDevice");
  if (rc != AQ_OK) return rc;
  static int sm_counts[64] = {0};
  if (sm_counts[device & 63] == 0) {
    int value = 0;
    rc = check_cuda(cudaDeviceGetAttribute(&value, cudaDevAttrMultiProcessorCount, device), "cudaDeviceGetAttribute");
    if (rc != AQ_OK) return rc;
    sm_counts[device & 63] = value;
  }
  *count = sm_counts[device & 63];
  return AQ_OK;
}

// Kernel variant of a problem: AQ_GEMM_TILE_WIDE (256 columns, one CTA per SM),
// AQ_GEMM_TILE_NARROW (128 columns, one CTA per SM) or AQ_GEMM_TILE_PAIRED (128 columns, two CTAs
// per SM), unless AQ_OPT_GEMM_TILE forces one.  K ranges over a cluster use the one-CTA-per-SM
// layouts (their exchange tile lives in the larger stage ring).
int tile_variant(int64_t m, int n_j, int split, int sm_count) {
  const int forced = gemm_tile_option();
  if (forced == AQ_GEMM_TILE_WIDE || forced == AQ_GEMM_TILE_NARROW) return forced;
  if (forced == AQ_GEMM_TILE_PAIRED) return split > 1 ? AQ_GEMM_TILE_NARROW : AQ_GEMM_TILE_PAIRED;
  if (split > 1) {
    const int64_t wide_ctas = ((m + kBM - 1) / kBM) * ((n_j + 3) / 4);
    return 2 * wide_ctas <= sm_count ? AQ_GEMM_TILE_NARROW : AQ_GEMM_TILE_WIDE;
  }
  return AQ_GEMM_TILE_PAIRED;
}

}  // namespace

int64_t tmem_gemm_workspace_bytes(int64_t, int, int) { return 0; }

// Number of K ranges (cluster size along z): more than one only where the output tiles alone
// would leave at least half of the SMs idle (few rows), at least four K steps per range.
// AQ_OPT_GEMM_SPLIT forces a value (for tests and measurements).
int tmem_gemm_split(int64_t m, int n_j, int n_k) {
  int sm_count = 148;
  if (device_sm_count(&sm_count) != AQ_OK) sm_count = 148;
  int split = gemm_split_option();
  if (split < 1 || split > 8) {
    split = 1;
    const int64_t wide_ctas = ((m + kBM - 1) / kBM) * ((n_j + 3) / 4);
    const int tn = 2 * wide_ctas <= sm_count ? 2 : 4;
    const int64_t ctas = ((m + kBM - 1) / kBM) * ((n_j + tn - 1) / tn);
    if (2 * ctas <= sm_count) split = static_cast<int>(sm_count / ctas < 8 ? sm_count / ctas : 8);
  }
  while (split > 1 && n_k / split < 4) --split;
  return split;
}

int launch_tmem_gemm(const LinearArgs& a, cudaStream_t stream) {
  if (a.n_k > kMaxNk) {
    return fail(AQ_ERR_INVALID, "the GEMM kernel supports K up to %d, got %d", kMaxNk * kTile,
                a.n_k * kTile);
  }
  int device = 0;
  int rc = check_cuda(cudaGetDevice(&device), "cudaGetDevice");
  if (rc != AQ_OK) return rc;
  int sm_count = 0;
  rc = device_sm_count(&sm_count);
  if (rc != AQ_OK) return rc;
  if (a.m >= (1LL << 31)) return fail(AQ_ERR_INVALID, "the GEMM kernel supports fewer than 2^31 rows");
  alignas(64) CUtensorMap x_map;
  rc = encode_activation_map(&x_map, a.xq, a.m, static_cast<int64_t>(a.n_k) * kTile, kBM);
  if (rc != AQ_OK) return rc;
  GemmParams p;
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
  const bool dump = a.acc_dump != nullptr;
  const bool fused = !gemm_separate_rounding();
  const int split = tmem_gemm_split(a.m, a.n_j, a.n_k);
  switch (tile_variant(a.m, a.n_j, split, sm_count)) {
    case AQ_GEMM_TILE_WIDE:
      return launch_shape<4, false>(x_map, p, dump, fused, split, device, stream);
    case AQ_GEMM_TILE_NARROW:
      return launch_shape<2, false>(x_map, p, dump, fused, split, device, stream);
    default:
      return launch_shape<2, true>(x_map, p, dump, fused, split, device, stream);
  }
}

int take_gemm_status() {
  int status = 0;
  if (cudaMemcpyFromSymbol(&status, g_gemm_status, sizeof(int)) != cudaSuccess) return -1;
  if (status != 0) {
    const int zero = 0;
    cudaMemcpyToSymbol(g_gemm_status, &zero, sizeof(int));
  }
  return status;
}

}  // namespace aq
