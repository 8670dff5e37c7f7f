// Mixed W4/W8 x A8 GEMM for large row counts on the Blackwell tensor cores (sm_100a).
//
// One CTA computes a 128-row x 256-column output tile (four 64-column weight tile
// rows) and walks K in 64-wide steps.  Per step:
//   * one elected thread streams the step's weight tiles from the prepared image into
//     shared memory with bulk asynchronous copies (cp.async.bulk, completion counted
//     on an mbarrier); a W8 tile is already in the 64-byte-swizzled K-major operand
//     layout and lands in place with one copy, W4 tiles land packed in a staging area;
//   * the producer warp copies the 128 x 64 int8 activation block with 16-byte
//     cp.async into the same K-major "core matrix" layout (8 rows x 16 bytes);
//   * two warps widen staged W4 tiles to int8 (value 16*w: one shift, one mask) into
//     the operand layout and publish them to the asynchronous proxy;
//   * one thread issues tcgen05.mma kind::i8 (M=128, N<=256, K=32, twice per step)
//     into one of two 256-column tensor-memory accumulators and commits to mbarriers;
//   * eight drain warps read the int32 accumulator with tcgen05.ld, turn it into FP32,
//     scale by (activation scale * tile scale) and add into FP32 registers -- integer
//     accumulation never spans two K64 tiles because every tile has its own scale
//     (operation order of alignquant/kernels/cuda/linear.cu:951-963).  The accumulators
//     are preset (tcgen05.st) to the bit pattern of 1.5 * 2^23, so the int32 result read
//     as a float is exactly 1.5 * 2^23 + sum and one exact FP32 subtraction stands in
//     for the much slower integer-to-float conversion.
// The epilogue stages rows through shared memory so that global stores are coalesced
// and applies the inverse output transform (linear.cu:983-1040) where a tile has one.
//
// Every mbarrier wait is bounded; on a time-out the CTA raises a device status word
// (read by aq_device_status), drains what it issued, frees its tensor memory and
// returns instead of hanging.
#include <mutex>

#include "aq_common.cuh"
#include "aq_ptx.cuh"
#include "aq_tile_math.cuh"

namespace aq {

__device__ int g_gemm_status = 0;

namespace {

constexpr int kBM = 128;
constexpr int kTilesN = 4;
constexpr int kStages = 4;
constexpr int kLag = 2;  // activation copies are published this many steps late
constexpr int kABytes = kBM * kTile;                 // 8192
constexpr int kBBytes = kTilesN * kW8TileBytes;      // 16384
constexpr int kPBytes = kTilesN * kW4TileBytes;      // 8192
constexpr int kStageBytes = kABytes + kBBytes + kPBytes;
constexpr int kMaxNk = 512;
constexpr int kRecBytes = kTilesN * kMaxNk * static_cast<int>(sizeof(TileRecord));
constexpr int kNumBars = 4 * kStages + 5;
constexpr int kSmemBytes = kStages * kStageBytes + kRecBytes + 512;
constexpr int kThreads = 384;
constexpr int kEpiRowFloats = 65;

struct GemmParams {
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

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, uint32_t src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes)
               : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
               : "memory");
}
__device__ __forceinline__ void tc_mma_i8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                          uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u)
      : "memory");
}
__device__ __forceinline__ void tc_ld32(uint32_t taddr, int (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]),
        "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]),
        "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]),
        "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]),
        "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tc_ld16(uint32_t taddr, int (&v)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]),
        "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]),
        "=r"(v[14]), "=r"(v[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// Store one 32-bit value into 16 consecutive columns of this warp's 32 tensor-memory lanes.
__device__ __forceinline__ void tc_st16(uint32_t taddr, const uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr),
      "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]),
      "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
      : "memory");
}

// The int32 accumulators start every K step at kBiasBits instead of zero.  Read back as
// an IEEE float, kBiasBits + d is exactly kBiasFloat + d for |d| < 2^22 (tile sums stay
// below 2^21 in magnitude, 16x-scaled W4 sums included), so one exact FP32 subtraction
// replaces the integer-to-float conversion, which runs at a quarter of the FP32 rate.
constexpr uint32_t kBiasBits = 0x4B400000u;  // 12582912.0f = 1.5 * 2^23
constexpr float kBiasFloat = 12582912.0f;

// K-major shared-memory operand descriptor.  Without swizzle the operand is made of
// 8-row x 16-byte core matrices: LBO = byte step between the two 16-byte K chunks of one
// MMA, SBO = byte step between 8-row groups.  With the 64-byte swizzle a row is 64
// contiguous bytes whose 16-byte chunks are XOR-ed with address bits 7-8, SBO is the
// step between 8-row groups (512 B) and LBO is not used (encoded as 16 B).
constexpr uint32_t kSwizzle64 = 4;
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo, uint32_t sbo, uint32_t layout) {
  return static_cast<uint64_t>((addr & 0x3ffffu) >> 4) |
         (static_cast<uint64_t>((lbo >> 4) & 0x3fffu) << 16) |
         (static_cast<uint64_t>((sbo >> 4) & 0x3fffu) << 32) | (1ull << 46) |
         (static_cast<uint64_t>(layout) << 61);
}
// kind::i8: D = S32 (2), A = B = signed 8-bit (1), both K-major, M = 128.
__device__ __forceinline__ uint32_t instr_desc_i8(int n) {
  return (2u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(n >> 3) << 17) |
         (static_cast<uint32_t>(kBM >> 4) << 24);
}

// acc[16*C .. 16*C+15] += float(d) * scale with d = v - kBiasBits; the subtraction is exact,
// multiply and add are rounded separately
template <int C>
__device__ __forceinline__ void drain_chunk(float (&acc)[128], const int (&v)[16], float scale) {
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const float d = __fadd_rn(__int_as_float(v[i]), -kBiasFloat);
    acc[C * 16 + i] = __fadd_rn(acc[C * 16 + i], __fmul_rn(d, scale));
  }
}

// Debug aid: the exact integer tile sums (W4 tiles were fed 16*w to the MMA).
__device__ __forceinline__ void dump_chunk(int32_t* tile_dump, int first_col, const int (&v)[16], const TileRecord& r) {
  if (tile_dump == nullptr) return;
  const int shift = (r.offset_flag & kW4Flag) ? 4 : 0;
  constexpr int kBias = static_cast<int>(kBiasBits);
  int4* o = reinterpret_cast<int4*>(tile_dump + first_col);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    o[i] = make_int4((v[4 * i] - kBias) >> shift, (v[4 * i + 1] - kBias) >> shift, (v[4 * i + 2] - kBias) >> shift,
                     (v[4 * i + 3] - kBias) >> shift);
  }
}

template <bool kDump>
__global__ void __launch_bounds__(kThreads, 1) tmem_gemm_kernel(const GemmParams p) {
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* stages = smem;
  TileRecord* rec_smem = reinterpret_cast<TileRecord*>(smem + kStages * kStageBytes);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kStages * kStageBytes + kRecBytes);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + kNumBars);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int n_k = p.n_k;
  const int j0 = blockIdx.x * kTilesN;
  const int tiles_here = min(kTilesN, p.n_j - j0);
  const int64_t m0 = static_cast<int64_t>(blockIdx.y) * kBM;
  const int64_t k_bytes = static_cast<int64_t>(n_k) * kTile;

  const uint32_t bar0 = smem_u32(bars);
  auto raw_full = [&](int s) { return bar0 + 8u * s; };
  auto a_full = [&](int s) { return bar0 + 8u * (kStages + s); };
  auto unpacked = [&](int s) { return bar0 + 8u * (2 * kStages + s); };
  auto empty = [&](int s) { return bar0 + 8u * (3 * kStages + s); };
  auto acc_full = [&](int b) { return bar0 + 8u * (4 * kStages + b); };
  auto acc_empty = [&](int b) { return bar0 + 8u * (4 * kStages + 2 + b); };
  const uint32_t final_bar = bar0 + 8u * (4 * kStages + 4);

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(raw_full(s), 1);
      mbar_init(a_full(s), 32);
      mbar_init(unpacked(s), 64);
      mbar_init(empty(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(acc_full(b), 1);
      mbar_init(acc_empty(b), 256);
    }
    mbar_init(final_bar, 1);
    *abort_flag = 0;
    mbar_init_fence();
    fence_proxy_async();
  }
  for (int i = threadIdx.x; i < tiles_here * n_k; i += kThreads) {
    const int t = i / n_k, kt = i % n_k;
    rec_smem[t * kMaxNk + kt] = p.records[static_cast<int64_t>(j0 + t) * n_k + kt];
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(tmem_slot)),
                 "r"(512u)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp < 4) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
    if (warp == 0) {
      // ---------------- producer: weights (bulk copies) + activations (cp.async) --
      int issued = 0;
      for (int kt = 0; kt < n_k; ++kt) {
        const int s = kt % kStages;
        const uint32_t ph = (kt / kStages) & 1;
        if (!mbar_wait(empty(s), ph ^ 1u, abort_flag, &g_gemm_status, 1)) break;
        uint8_t* a_s = stages + s * kStageBytes;
        const uint32_t a_addr = smem_u32(a_s);
        const uint32_t b_addr = a_addr + kABytes;
        const uint32_t p_addr = b_addr + kBBytes;
        if (lane == 0) {
          uint32_t bytes = 0;
          for (int t = 0; t < tiles_here; ++t) {
            bytes += (rec_smem[t * kMaxNk + kt].offset_flag & kW4Flag) ? kW4TileBytes : kW8TileBytes;
          }
          mbar_expect_tx(raw_full(s), bytes);
          for (int t = 0; t < tiles_here; ++t) {
            const uint32_t of = rec_smem[t * kMaxNk + kt].offset_flag;
            const uint8_t* src = p.payload + static_cast<int64_t>(of & ~kW4Flag) * kW4TileBytes;
            if (of & kW4Flag) {
              bulk_copy(p_addr + t * kW4TileBytes, src, kW4TileBytes, raw_full(s));
            } else {
              bulk_copy(b_addr + t * kW8TileBytes, src, kW8TileBytes, raw_full(s));
            }
          }
        }
#pragma unroll 4
        for (int i = 0; i < 16; ++i) {
          const int q = lane + 32 * i;
          const int row = q >> 2, c = q & 3;
          const int64_t grow = m0 + row;
          const bool valid = grow < p.m;
          const int8_t* src = p.xq + (valid ? grow : 0) * k_bytes + static_cast<int64_t>(kt) * kTile + c * 16;
          cp_async16(a_addr + c * 2048 + (row >> 3) * 128 + (row & 7) * 16, src, valid ? 16u : 0u);
        }
        cp_async_commit();
        issued = kt + 1;
        if (kt >= kLag) {
          cp_async_wait<kLag>();
          fence_proxy_async();
          mbar_arrive(a_full((kt - kLag) % kStages));
        }
      }
      cp_async_wait<0>();
      fence_proxy_async();
      for (int kt = max(0, issued - kLag); kt < issued; ++kt) mbar_arrive(a_full(kt % kStages));
      if (*abort_flag != 0 && lane == 0) {
        // give bulk copies still in flight a bounded chance to land before the CTA exits
        for (int kt = max(0, issued - kStages); kt < issued; ++kt) {
          const uint32_t bar = raw_full(kt % kStages);
          for (uint32_t i = 0; i < (1u << 16) && !mbar_try_wait(bar, (kt / kStages) & 1); ++i) {
          }
        }
      }
    } else if (warp == 1) {
      // ---------------- MMA issuer -------------------------------------------------
      if (lane == 0) {
        const uint32_t idesc = instr_desc_i8(64 * tiles_here);
        bool ok = true;
        for (int kt = 0; kt < n_k && ok; ++kt) {
          const int s = kt % kStages;
          const uint32_t ph = (kt / kStages) & 1;
          const int b = kt & 1;
          const uint32_t pha = (kt >> 1) & 1;
          ok = mbar_wait(raw_full(s), ph, abort_flag, &g_gemm_status, 2) && mbar_wait(a_full(s), ph, abort_flag, &g_gemm_status, 3) &&
               mbar_wait(unpacked(s), ph, abort_flag, &g_gemm_status, 4) &&
               mbar_wait(acc_empty(b), pha, abort_flag, &g_gemm_status, 5);
          if (!ok) break;
          tc_fence_after();
          const uint32_t a_addr = smem_u32(stages + s * kStageBytes);
          const uint32_t b_addr = a_addr + kABytes;
          const uint32_t d = tmem_base + static_cast<uint32_t>(b) * 256u;
          // A: no swizzle, 16-byte K chunks 2048 B apart, 8-row groups 128 B apart.
          // B: 64-byte swizzle, rows of 64 B, 8-row groups 512 B apart; the second K32
          // half of a row starts 32 B further on.
          // the accumulator was preset to kBiasBits by the drain warps: always accumulate
          tc_mma_i8(d, smem_desc(a_addr, 2048, 128, 0), smem_desc(b_addr, 16, 512, kSwizzle64), idesc, 1u);
          tc_mma_i8(d, smem_desc(a_addr + 4096, 2048, 128, 0), smem_desc(b_addr + 32, 16, 512, kSwizzle64), idesc, 1u);
          tc_commit(empty(s));
          tc_commit(acc_full(b));
        }
        if (!ok) {
          // make sure nothing issued is still running before tensor memory is freed
          tc_commit(final_bar);
          for (uint32_t i = 0; i < (1u << 20) && !mbar_try_wait(final_bar, 0); ++i) {
          }
        }
      }
      __syncwarp();
    } else {
      // ---------------- W4 widening: packed staging -> int8 operand layout ---------
      const int u = threadIdx.x - 64;
      for (int kt = 0; kt < n_k; ++kt) {
        const int s = kt % kStages;
        const uint32_t ph = (kt / kStages) & 1;
        if (!mbar_wait(raw_full(s), ph, abort_flag, &g_gemm_status, 6)) break;
        uint8_t* b_s = stages + s * kStageBytes + kABytes;
        const uint8_t* p_s = b_s + kBBytes;
        for (int t = 0; t < tiles_here; ++t) {
          if (rec_smem[t * kMaxNk + kt].offset_flag & kW4Flag) {
#pragma unroll
            for (int rep = 0; rep < 2; ++rep) {
              // packed chunk q = 2*n + h: low nibbles are k16 block 2h of row n, high nibbles 2h+1
              const int q = rep * 64 + u;
              const int n = q >> 1, h = q & 1;
              const uint4 pk = *reinterpret_cast<const uint4*>(p_s + t * kW4TileBytes + q * 16);
              uint4 lo, hi;
              lo.x = (pk.x << 4) & 0xf0f0f0f0u;
              lo.y = (pk.y << 4) & 0xf0f0f0f0u;
              lo.z = (pk.z << 4) & 0xf0f0f0f0u;
              lo.w = (pk.w << 4) & 0xf0f0f0f0u;
              hi.x = pk.x & 0xf0f0f0f0u;
              hi.y = pk.y & 0xf0f0f0f0u;
              hi.z = pk.z & 0xf0f0f0f0u;
              hi.w = pk.w & 0xf0f0f0f0u;
              uint8_t* row = b_s + t * kW8TileBytes + n * 64;
              const int swz = (n >> 1) & 3;
              *reinterpret_cast<uint4*>(row + (((2 * h) ^ swz) << 4)) = lo;
              *reinterpret_cast<uint4*>(row + (((2 * h + 1) ^ swz) << 4)) = hi;
            }
          }
        }
        fence_proxy_async();
        mbar_arrive(unpacked(s));
      }
    }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 224;");
    // ---------------- drain: int32 accumulator -> scaled FP32 registers -------------
    const int quarter = warp & 3;       // tensor-memory lane quarter this warp may read
    const int half = (warp - 4) >> 2;   // column half: weight tile rows 2*half, 2*half+1
    const int row = quarter * 32 + lane;
    const int64_t grow = m0 + row;
    const bool row_valid = grow < p.m;
    const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                           static_cast<uint32_t>(half * 128);
    float acc[128];
#pragma unroll
    for (int i = 0; i < 128; ++i) acc[i] = 0.0f;
    const float token_scale =
        (p.scale_mode == AQ_SCALE_TOKEN && row_valid) ? p.act_scales[grow] : 0.0f;
    const float* tile_scales =
        (p.scale_mode == AQ_SCALE_TILE && row_valid) ? p.act_scales + (grow >> 4) * n_k : nullptr;
    const TileRecord* rec_lo = rec_smem + (2 * half) * kMaxNk;
    const TileRecord* rec_hi = rec_lo + kMaxNk;

    // Software pipeline over 16-column chunks (four per weight tile, eight per K step) with
    // two register buffers: while the FP32 work of one chunk runs, the tensor-memory load of
    // the next one is in flight.  A chunk's columns are preset again right after they have been
    // read, and the accumulator goes back to the MMA thread as soon as its last chunk has been
    // loaded, before that chunk's arithmetic.
    int va[16], vb[16];
    uint32_t bias[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) bias[i] = kBiasBits;
    // preset this warp's part of both accumulators, then hand them to the MMA thread
#pragma unroll
    for (int c = 0; c < 16; ++c) tc_st16(taddr + static_cast<uint32_t>((c >> 3) * 256 + (c & 7) * 16), bias);
    tc_wait_st();
    tc_fence_before();
    mbar_arrive(acc_empty(0));
    mbar_arrive(acc_empty(1));
    bool ok = mbar_wait(acc_full(0), 0, abort_flag, &g_gemm_status, 7);
    if (ok) {
      tc_fence_after();
      tc_ld16(taddr, va);
    }
    for (int kt = 0; kt < n_k && ok; ++kt) {
      const int b = kt & 1;
      const uint32_t col = taddr + static_cast<uint32_t>(b * 256);
      const float a_scale = tile_scales != nullptr ? tile_scales[kt] : token_scale;
      const TileRecord r0 = rec_lo[kt];
      const TileRecord r1 = rec_hi[kt];
      const float s0 = __fmul_rn(a_scale, r0.scale);
      const float s1 = __fmul_rn(a_scale, r1.scale);
      int32_t* dump0 = nullptr;
      int32_t* dump1 = nullptr;
      if (kDump && row_valid) {
        if (2 * half < tiles_here) dump0 = p.acc_dump + ((grow * p.n_j + (j0 + 2 * half)) * n_k + kt) * kTile;
        if (2 * half + 1 < tiles_here) dump1 = p.acc_dump + ((grow * p.n_j + (j0 + 2 * half + 1)) * n_k + kt) * kTile;
      }
#define AQ_DRAIN_STEP(C, CUR, NEXT, SCALE, DUMP, REC)                 \
      tc_wait_ld();                                                  \
      tc_st16(col + (C) * 16, bias);                                 \
      tc_ld16(col + ((C) + 1) * 16, NEXT);                           \
      drain_chunk<C>(acc, CUR, SCALE);                               \
      if (kDump) dump_chunk(DUMP, ((C) & 3) * 16, CUR, REC);
      AQ_DRAIN_STEP(0, va, vb, s0, dump0, r0)
      AQ_DRAIN_STEP(1, vb, va, s0, dump0, r0)
      AQ_DRAIN_STEP(2, va, vb, s0, dump0, r0)
      AQ_DRAIN_STEP(3, vb, va, s0, dump0, r0)
      AQ_DRAIN_STEP(4, va, vb, s1, dump1, r1)
      AQ_DRAIN_STEP(5, vb, va, s1, dump1, r1)
      AQ_DRAIN_STEP(6, va, vb, s1, dump1, r1)
#undef AQ_DRAIN_STEP
      tc_wait_ld();  // chunk 7 in vb: this accumulator has been read completely
      tc_st16(col + 7 * 16, bias);
      tc_wait_st();
      tc_fence_before();
      mbar_arrive(acc_empty(b));
      if (kt + 1 < n_k) {
        ok = mbar_wait(acc_full(b ^ 1), ((kt + 1) >> 1) & 1, abort_flag, &g_gemm_status, 7);
        if (ok) {
          tc_fence_after();
          tc_ld16(taddr + static_cast<uint32_t>((b ^ 1) * 256), va);
        }
      }
      drain_chunk<7>(acc, vb, s1);
      if (kDump) dump_chunk(dump1, 48, vb, r1);
    }

    // ---------------- epilogue: rows through shared memory, coalesced stores --------
    if (ok) {
      float* region = reinterpret_cast<float*>(stages) + (warp - 4) * (32 * kEpiRowFloats);
      const int64_t n_cols = static_cast<int64_t>(p.n_j) * kTile;
#pragma unroll
      for (int t = 0; t < 2; ++t) {
        const int tl = 2 * half + t;
        if (tl < tiles_here) {
          const int j = j0 + tl;
#pragma unroll
          for (int c = 0; c < 64; ++c) region[lane * kEpiRowFloats + c] = acc[t * 64 + c];
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

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u)
                 : "memory");
  }
}

std::once_flag g_attr_once[64];

}  // namespace

int64_t tmem_gemm_workspace_bytes(int64_t, int, int) { return 0; }

int launch_tmem_gemm(const LinearArgs& a, cudaStream_t stream) {
  if (a.n_k > kMaxNk) {
    return fail(AQ_ERR_INVALID, "the GEMM kernel supports K up to %d, got %d", kMaxNk * kTile,
                a.n_k * kTile);
  }
  int device = 0;
  int rc = check_cuda(cudaGetDevice(&device), "cudaGetDevice");
  if (rc != AQ_OK) return rc;
  cudaError_t attr_status = cudaSuccess;
  std::call_once(g_attr_once[device & 63], [&] {
    attr_status = cudaFuncSetAttribute(tmem_gemm_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       kSmemBytes);
    if (attr_status == cudaSuccess) {
      attr_status = cudaFuncSetAttribute(tmem_gemm_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         kSmemBytes);
    }
  });
  rc = check_cuda(attr_status, "cudaFuncSetAttribute(tmem_gemm_kernel)");
  if (rc != AQ_OK) return rc;
  GemmParams p;
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
  const dim3 grid(static_cast<unsigned>((a.n_j + kTilesN - 1) / kTilesN),
                  static_cast<unsigned>((a.m + kBM - 1) / kBM));
  if (a.acc_dump != nullptr) {
    tmem_gemm_kernel<true><<<grid, kThreads, kSmemBytes, stream>>>(p);
  } else {
    tmem_gemm_kernel<false><<<grid, kThreads, kSmemBytes, stream>>>(p);
  }
  return check_cuda(cudaGetLastError(), "tensor-memory GEMM launch");
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
