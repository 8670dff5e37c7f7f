// Decode kernel for at most 32 rows without a shared-memory ring, mbarriers or a split-K
// exchange between CTAs: many small CTAs that fetch their whole weight block at once.
//
// A decode-size projection is one to five microseconds of HBM traffic, so what a kernel costs
// is its chain of latencies, not its bytes, and what a chain of such kernels costs is how much
// of one kernel's chain hides behind the previous kernel.  This kernel is built for that:
//   * one CTA per (tile row j, group of 16 -- or 8 -- output columns q).  The rows of a column
//     group are one contiguous block of a tile of the prepared image (1 KiB of a W8 tile, 512 B
//     of a W4 tile for 16 columns), and lane (g, c) of a warp needs exactly two 16-byte vectors
//     of it (columns g and g + 8, k in [16c, 16c + 16)): the operand layout of
//     mma.sync.m16n8k32.s8 with the weights as the 16-row operand and up to eight activation
//     rows as the 8-column operand;
//   * warp w owns the tiles k = w, w + WARPS, ... of the row.  BEFORE the grid dependency is
//     resolved (weights are static) every lane copies all its vectors of all its tiles into
//     shared memory with 16-byte asynchronous copies (cp.async): the whole block of the CTA, a
//     few tens of KiB, is requested at once, by coalesced 128-bit accesses, and costs no
//     registers while it is in flight.  A CTA is small (four or eight warps, its block of
//     shared memory), so the CTAs of the next one or two launches are resident, with their
//     weights on the way or landed, while the current launch still runs;
//   * after the dependency only the activations are missing: their vectors go straight into
//     registers (up to twelve tiles ahead), then MMAs from shared memory, per-tile scaling,
//     and ONE CTA barrier: K is not split over CTAs, the warp sums meet in a few KiB of shared
//     memory and COLS x rows values are stored.  Only a tile row with a non-identity output
//     transform needs its column groups together: such launches run as clusters that exchange
//     their columns through distributed shared memory.
// Under tensor parallelism the thread that finishes a value also sums it over the ranks: it
// stores the value, tagged with the number of the call, into every peer's receive area (plain
// NVLink stores), polls the peers' units of the same position in its own receive area (bounded)
// and adds in rank order -- the protocol of aq_allreduce.cu without a second launch.
//
// Summation order (all FP32, separately rounded multiply and add as in
// alignquant/kernels/cuda/linear.cu:956-963): warp w adds its tiles in increasing k, the warp
// sums are added in warp order -- aq_linear_plan reports one K range and WARPS workers.
#include <cooperative_groups.h>

#include <mutex>

#include "aq_common.cuh"
#include "aq_ptx.cuh"
#include "aq_quantize_math.cuh"
#include "aq_tile_math.cuh"

namespace cg = cooperative_groups;

namespace aq {
namespace {

struct DirectParams {
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
  const uint8_t* prefetch;
  int64_t prefetch_bytes;
  // kQuant: the activations arrive as fp16 / bf16 rows and are quantized by the kernel; xq and
  // act_scales then receive the int8 rows and their scales (written by one CTA)
  const void* raw_x;
  int raw_bf16;
  // fused sum over tensor-parallel ranks (tp_world <= 1: off)
  ArPeers peers;
  int tp_rank;
  int tp_world;
  int64_t ar_max_count;
  uint32_t ar_poll_limit;
};

__device__ int g_direct_decode_status = 0;

// One exchange unit {value, call number} as ONE 64-bit scalar access: a 64-bit access is
// single-copy atomic, so a reader never sees a new tag with an old value (a two-element vector
// access would be two scalar accesses in unspecified order by the memory model).
__device__ __forceinline__ void st_volatile_v2(void* p, uint32_t a, uint32_t b) {
  const uint64_t unit = static_cast<uint64_t>(a) | (static_cast<uint64_t>(b) << 32);
  asm volatile("st.volatile.global.u64 [%0], %1;" ::"l"(p), "l"(unit) : "memory");
}
__device__ __forceinline__ uint2 ld_volatile_v2(const void* p) {
  uint64_t unit;
  asm volatile("ld.volatile.global.u64 %0, [%1];" : "=l"(unit) : "l"(p) : "memory");
  return make_uint2(static_cast<uint32_t>(unit), static_cast<uint32_t>(unit >> 32));
}

// This rank's finished value of output element `e` -> the sum over the ranks, in rank order.
__device__ __forceinline__ float sum_over_ranks(const DirectParams& p, uint32_t epoch, int64_t e, float own) {
  const int64_t area = (static_cast<int64_t>(epoch & 1u) * p.tp_world) * p.ar_max_count;  // values
  for (int step = 1; step < p.tp_world; ++step) {
    const int peer = (p.tp_rank + step) % p.tp_world;  // every rank starts with a different peer
    st_volatile_v2(p.peers.buffer[peer] + kArHeaderBytes + (area + p.tp_rank * p.ar_max_count + e) * 8,
                   __float_as_uint(own), epoch);
  }
  // The peers' units are requested together and re-requested only where the tag is still old: one
  // L2 round trip for all ranks that have delivered, not one per rank (measured: the sum cost
  // about 0.85 us per rank when the loads were issued one after the other).
  const uint8_t* const mine = p.peers.buffer[p.tp_rank] + kArHeaderBytes + (area + e) * 8;
  const int64_t rank_stride = p.ar_max_count * 8;
  uint2 unit[kArMaxRanks];
#pragma unroll
  for (int r = 0; r < kArMaxRanks; ++r) {
    unit[r] = make_uint2(0u, epoch);
    if (r < p.tp_world && r != p.tp_rank) unit[r] = ld_volatile_v2(mine + r * rank_stride);
  }
  for (uint32_t polls = 0;;) {
    bool complete = true;
#pragma unroll
    for (int r = 0; r < kArMaxRanks; ++r) {
      if (unit[r].y != epoch) {
        complete = false;
        unit[r] = ld_volatile_v2(mine + r * rank_stride);
      }
    }
    if (complete) break;
    if (++polls >= p.ar_poll_limit) {
      int late = 0;
#pragma unroll
      for (int r = 0; r < kArMaxRanks; ++r) late = (unit[r].y != epoch && late == 0) ? 40 + r : late;
      if (late != 0) atomicCAS(&g_direct_decode_status, 0, late);
      break;
    }
    if (polls > 64) __nanosleep(100);
  }
  float total = 0.0f;
#pragma unroll
  for (int r = 0; r < kArMaxRanks; ++r) {
    if (r < p.tp_world) {
      const float v = r == p.tp_rank ? own : __uint_as_float(unit[r].x);
      total = r == 0 ? v : __fadd_rn(total, v);
    }
  }
  return total;
}

// 16 bytes global -> shared, asynchronous, not kept in L1
__device__ __forceinline__ void copy16_async(uint32_t dst, const uint8_t* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void copy_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }
__device__ __forceinline__ void sts16(uint32_t addr, const uint4& v) {
  asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ uint4 lds16(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}

// Rows up to which the kernel quantizes its own activations (kQuant).  Every CTA rounds the whole
// row, so the work is replicated on every SM: at one row that costs less than the quantizer launch
// it replaces (3072 x 1536: 3.4 against 4.3 us per pair), at four rows far more (6.3 against 4.6 us).
constexpr int kQuantRows = 1;

// Bytes of a warp's block of shared memory: its tiles' weights, and room for its sums afterwards.
__host__ __device__ constexpr uint32_t warp_block_bytes(int tiles_per_warp, int block_bytes, int sums_bytes) {
  return static_cast<uint32_t>(tiles_per_warp * block_bytes > sums_bytes ? tiles_per_warp * block_bytes : sums_bytes);
}

// NG: groups of eight activation rows (1, 2 or 4).  COLS: output columns of a CTA (16 or 8).
// WARPS: warps of a CTA.  kCluster: launched as clusters of the 64 / COLS column groups of a tile
// row (layers that carry an output transform).  kTp: the finished values are also summed over
// the tensor-parallel ranks.  kQuant (one row): the kernel is also the per-token
// activation quantizer -- every CTA needs all of every row anyway, so it finds the rows' maxima and
// rounds the rows into its shared memory itself, with the quantizer kernel's own arithmetic; the
// separate quantizer launch, its dependency latency and one round trip through the L2 go away.
template <int NG, int COLS, int WARPS, bool kCluster, bool kTp, bool kQuant>
__global__ void __launch_bounds__(32 * WARPS, NG == 1 ? 3 : 2) direct_decode_kernel(const DirectParams p) {
  constexpr int kRows = 8 * NG;
  constexpr int kThreads = 32 * WARPS;
  constexpr int kGroups = kTile / COLS;
  constexpr int kBlockBytes = COLS * kTile;  // a W8 column group of one tile; W4 takes the first half
  // [WARPS][tiles per warp][kBlockBytes], then the activation rows.  A warp's block of weights
  // becomes its [kRows][COLS] sums once its loop is over (nobody else reads the block).
  extern __shared__ __align__(128) uint8_t staged[];
  __shared__ float finished[kRows][COLS];  // the CTA's columns, read by its cluster peers
  __shared__ uint32_t epoch_shared;
  __shared__ float row_max_part[kQuant ? kQuantRows : 1][WARPS];
  __shared__ float row_scale[kQuant ? kQuantRows : 1];

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int g = lane >> 2;
  const int c = lane & 3;
  const int j = blockIdx.x;
  const int q = blockIdx.y;
  const int n_k = p.n_k;
  const int rows = p.m < kRows ? static_cast<int>(p.m) : kRows;
  const int tiles_per_warp = (n_k + WARPS - 1) / WARPS;
  const uint32_t warp_stage_bytes = warp_block_bytes(tiles_per_warp, kBlockBytes, kRows * COLS * 4);
  const int my_tiles = warp < n_k ? (n_k - warp + WARPS - 1) / WARPS : 0;  // tiles w, w + WARPS, ...

  grid_launch_dependents();

  // ---- before the grid dependency: the CTA's whole weight block goes to shared memory -----------
  // Lane t holds the record of the warp's tile t + 32 * chunk; every lane copies exactly the
  // 16-byte vectors it will read (the two lanes that share a W4 vector: the even one copies).
  const TileRecord* row_records = p.records + static_cast<int64_t>(j) * n_k;
  const uint32_t w8_off = static_cast<uint32_t>(g * 64 + ((c ^ ((g >> 1) & 3)) << 4));
  const uint32_t w4_off = static_cast<uint32_t>(g * 32 + (c >> 1) * 16);
  const int w4_shift = (c & 1) ? 0 : 4;
  const uint32_t my_stage = smem_u32(staged) + static_cast<uint32_t>(warp) * warp_stage_bytes;
  TileRecord lane_rec = {0u, 0.0f};
  for (int i = 0; i < my_tiles; ++i) {
    if ((i & 31) == 0) {
      lane_rec = {0u, 0.0f};
      if (i + lane < my_tiles) lane_rec = row_records[warp + WARPS * (i + lane)];
    }
    const uint32_t of = __shfl_sync(0xffffffffu, lane_rec.offset_flag, i & 31);
    const uint8_t* tile = p.payload + static_cast<int64_t>(of & ~kW4Flag) * kW4TileBytes;
    const uint32_t slot = my_stage + static_cast<uint32_t>(i) * kBlockBytes;
    if (of & kW4Flag) {
      if ((c & 1) == 0) {
        const uint8_t* block = tile + q * (COLS * 32) + w4_off;
        copy16_async(slot + w4_off, block);
        if (COLS == 16) copy16_async(slot + w4_off + 8 * 32, block + 8 * 32);
      }
    } else {
      const uint8_t* block = tile + q * (COLS * 64) + w8_off;
      copy16_async(slot + w8_off, block);
      if (COLS == 16) copy16_async(slot + w8_off + 8 * 64, block + 8 * 64);
    }
  }
  // Still before the dependency: wait for the block and widen its W4 tiles in place (every slot
  // has the size of a W8 block), so that after the dependency all tiles are read alike: two
  // vectors at fixed offsets, no selects, no shifts.  Every lane of a pair reads the packed
  // vector before any lane writes.
  copy_async_wait_all();
  __syncwarp();
  // The look-ahead for the next launch goes out behind this CTA's own weights, one piece per warp
  // at a time.  It pays where other kernels run between two projections; in a chain of nothing but
  // projections it was measured to cost more than it gives whenever it is issued (at the start,
  // here, or after the activation rows have landed).
  if (lane == 0 && p.prefetch_bytes > 0) {
    prefetch_slice_l2(p.prefetch, p.prefetch_bytes, static_cast<int64_t>(blockIdx.x) * gridDim.y + blockIdx.y,
                      static_cast<int64_t>(gridDim.x) * gridDim.y, warp, WARPS);
  }
  uint32_t w4_tiles = 0;  // bit i % 32: the warp's tile i is W4 (for the debug dump)
  if (my_tiles > 32) {
    lane_rec = {0u, 0.0f};
    if (lane < my_tiles) lane_rec = row_records[warp + WARPS * lane];
  }
  for (int i = 0; i < my_tiles; ++i) {
    if (i != 0 && (i & 31) == 0) {
      lane_rec = {0u, 0.0f};
      if (i + lane < my_tiles) lane_rec = row_records[warp + WARPS * (i + lane)];
    }
    const uint32_t of = __shfl_sync(0xffffffffu, lane_rec.offset_flag, i & 31);
    if (of & kW4Flag) {
      if (i < 32) w4_tiles |= 1u << i;
      const uint32_t slot = my_stage + static_cast<uint32_t>(i) * kBlockBytes;
      uint4 a = lds16(slot + w4_off);
      uint4 b = make_uint4(0, 0, 0, 0);
      if (COLS == 16) b = lds16(slot + w4_off + 8 * 32);
      __syncwarp();
      a.x = (a.x << w4_shift) & 0xf0f0f0f0u;
      a.y = (a.y << w4_shift) & 0xf0f0f0f0u;
      a.z = (a.z << w4_shift) & 0xf0f0f0f0u;
      a.w = (a.w << w4_shift) & 0xf0f0f0f0u;
      sts16(slot + w8_off, a);
      if (COLS == 16) {
        b.x = (b.x << w4_shift) & 0xf0f0f0f0u;
        b.y = (b.y << w4_shift) & 0xf0f0f0f0u;
        b.z = (b.z << w4_shift) & 0xf0f0f0f0u;
        b.w = (b.w << w4_shift) & 0xf0f0f0f0u;
        sts16(slot + w8_off + 8 * 64, b);
      }
    }
  }
  if (my_tiles > 32) {  // back to the first block of records for the scales below
    lane_rec = {0u, 0.0f};
    if (lane < my_tiles) lane_rec = row_records[warp + WARPS * lane];
  }
  __syncwarp();
  // Everything that can be computed from the kernel parameters is computed here: the first read
  // of a parameter after the dependency would cost a round trip of its own (parameters live in
  // constant memory, which the SM caches per line).
  const int64_t k_bytes = static_cast<int64_t>(n_k) * kTile;
  const uint32_t x_stride = static_cast<uint32_t>(k_bytes) + 64u;  // padded rows: no bank conflicts between rows
  const uint32_t x_stage = smem_u32(staged) + static_cast<uint32_t>(WARPS) * warp_stage_bytes;
  const int8_t* const x_global = p.xq;
  const float* const scale_global = p.act_scales;
  const bool token_mode = p.scale_mode == AQ_SCALE_TOKEN;
  int32_t* const dump_global = p.acc_dump;
  const uint4* const raw_global = static_cast<const uint4*>(p.raw_x);
  const bool raw_bf16 = p.raw_bf16 != 0;
  int8_t* const q_global = const_cast<int8_t*>(p.xq);
  float* const scale_out = const_cast<float*>(p.act_scales);
  const int chunks_per_row = n_k * 4;  // 16-byte pieces of an activation row

  grid_dependency_wait();  // activations and their scales come from the preceding kernel
  if (kTp && threadIdx.x == 0) {
    epoch_shared = *reinterpret_cast<const volatile uint32_t*>(p.peers.buffer[p.tp_rank]) + 1;  // number of this call
  }

  // ---- after it: the activation rows go to shared memory, then a short loop over the tiles -------
  float token_scale[NG][2];
  if (kQuant) {
    // Pass 1: the row's absolute maximum (16-byte vectors of eight values, all threads of the CTA).
    const int vectors_per_row = n_k * 8;
    for (int r = 0; r < rows; ++r) {
      float amax = 0.0f;
      for (int v = threadIdx.x; v < vectors_per_row; v += kThreads) {
        float f[8];
        unpack8(__ldg(raw_global + static_cast<int64_t>(r) * vectors_per_row + v), raw_bf16, f);
#pragma unroll
        for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(f[i]));
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
      if (lane == 0) row_max_part[r][warp] = amax;
    }
    __syncthreads();
    const bool writer = blockIdx.x == 0 && blockIdx.y == 0;  // one CTA leaves the int8 row and its scale to the caller
    if (threadIdx.x < rows) {
      float row_max = row_max_part[threadIdx.x][0];
#pragma unroll
      for (int w = 1; w < WARPS; ++w) row_max = fmaxf(row_max, row_max_part[threadIdx.x][w]);
      const float scale = token_scale_of(row_max);
      row_scale[threadIdx.x] = scale;
      if (writer) scale_out[threadIdx.x] = scale;
    }
    __syncthreads();
    // Pass 2: the same vectors again (they are in the L1 now), rounded into the staged int8 row.
    for (int r = 0; r < rows; ++r) {
      const float scale = row_scale[r];
      const float inv_scale = __fdiv_rn(1.0f, scale);
      for (int v = threadIdx.x; v < vectors_per_row; v += kThreads) {
        float f[8];
        unpack8(__ldg(raw_global + static_cast<int64_t>(r) * vectors_per_row + v), raw_bf16, f);
        int q8[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) q8[i] = quantize_token_value(f[i], scale, inv_scale);
        const uint32_t lo = pack4(q8[0], q8[1], q8[2], q8[3]), hi = pack4(q8[4], q8[5], q8[6], q8[7]);
        asm volatile("st.shared.v2.u32 [%0], {%1, %2};" ::"r"(x_stage + static_cast<uint32_t>(r) * x_stride + static_cast<uint32_t>(v) * 8u),
                     "r"(lo), "r"(hi)
                     : "memory");
        if (writer) *reinterpret_cast<uint2*>(q_global + static_cast<int64_t>(r) * k_bytes + v * 8) = make_uint2(lo, hi);
      }
    }
#pragma unroll
    for (int ng = 0; ng < NG; ++ng) {
      const int tok = ng * 8 + 2 * c;
      token_scale[ng][0] = tok < rows ? row_scale[tok < kQuantRows ? tok : 0] : 0.0f;
      token_scale[ng][1] = tok + 1 < rows ? row_scale[tok + 1 < kQuantRows ? tok + 1 : 0] : 0.0f;
    }
  } else {
    for (int t = threadIdx.x; t < rows * chunks_per_row; t += kThreads) {
      const int r = t / chunks_per_row, ck = t - r * chunks_per_row;
      copy16_async(x_stage + static_cast<uint32_t>(r) * x_stride + static_cast<uint32_t>(ck) * 16u,
                   reinterpret_cast<const uint8_t*>(x_global) + static_cast<int64_t>(r) * k_bytes + ck * 16);
    }
#pragma unroll
    for (int ng = 0; ng < NG; ++ng) {
      const int tok = ng * 8 + 2 * c;
      token_scale[ng][0] = (token_mode && tok < rows) ? scale_global[tok] : 0.0f;
      token_scale[ng][1] = (token_mode && tok + 1 < rows) ? scale_global[tok + 1] : 0.0f;
    }
  }
  copy_async_wait_all();
  __syncthreads();
  float acc[NG][4];
#pragma unroll
  for (int ng = 0; ng < NG; ++ng) acc[ng][0] = acc[ng][1] = acc[ng][2] = acc[ng][3] = 0.0f;

  // Per tile: two 16-byte reads of weights at fixed offsets, one of activations per row group,
  // two MMAs per row group, one shuffle for the tile's scale, and the scaled accumulation of the
  // tile before (the MMAs of a tile are in flight while the sums of the last one are added).  The
  // loop is rolled on purpose: every warp runs its body many times, so the instructions are fetched
  // once; unrolled over all tiles, instruction fetch, not arithmetic, set the pace.
  auto accumulate = [&](const int (&d)[NG][4], float w_s, int i) {
    const int kt = warp + WARPS * i;
#pragma unroll
    for (int ng = 0; ng < NG; ++ng) {
      float s0, s1;
      if (token_mode) {
        s0 = __fmul_rn(token_scale[ng][0], w_s);
        s1 = __fmul_rn(token_scale[ng][1], w_s);
      } else {
        // tokens 8*ng .. 8*ng+7 share the scale of their 16-row group
        const float a_s = (ng * 8 < rows) ? scale_global[static_cast<int64_t>(ng >> 1) * n_k + kt] : 0.0f;
        s0 = s1 = __fmul_rn(a_s, w_s);
      }
      acc[ng][0] = __fadd_rn(acc[ng][0], __fmul_rn(static_cast<float>(d[ng][0]), s0));
      acc[ng][1] = __fadd_rn(acc[ng][1], __fmul_rn(static_cast<float>(d[ng][1]), s1));
      if (COLS == 16) {
        acc[ng][2] = __fadd_rn(acc[ng][2], __fmul_rn(static_cast<float>(d[ng][2]), s0));
        acc[ng][3] = __fadd_rn(acc[ng][3], __fmul_rn(static_cast<float>(d[ng][3]), s1));
      }
      if (dump_global != nullptr) {
        const int shift = ((w4_tiles >> (i & 31)) & 1u) ? 4 : 0;
        const int tok = ng * 8 + 2 * c;
#pragma unroll
        for (int e = 0; e < (COLS == 16 ? 4 : 2); ++e) {
          const int t = tok + (e & 1);
          const int col = q * COLS + g + ((e & 2) ? 8 : 0);
          if (t < rows) {
            dump_global[((static_cast<int64_t>(t) * p.n_j + j) * n_k + kt) * kTile + col] = d[ng][e] >> shift;
          }
        }
      }
    }
  };

  uint32_t w_addr = my_stage + w8_off;                                              // this lane's vector of tile 0
  uint32_t x_addr = x_stage + static_cast<uint32_t>(g) * x_stride + static_cast<uint32_t>(warp * kTile + c * 16);
  bool x_row[NG];
#pragma unroll
  for (int ng = 0; ng < NG; ++ng) x_row[ng] = ng * 8 + g < rows;
  int d_prev[NG][4];
  float ws_prev = 0.0f;
#pragma unroll 2
  for (int i = 0; i < my_tiles; ++i) {
    if (i != 0 && (i & 31) == 0) {  // very long rows: the next block of 32 records
      lane_rec = {0u, 0.0f};
      if (i + lane < my_tiles) lane_rec = row_records[warp + WARPS * (i + lane)];
      w4_tiles = __ballot_sync(0xffffffffu, (lane_rec.offset_flag & kW4Flag) != 0);
    }
    const uint4 a = lds16(w_addr);
    uint4 b = make_uint4(0, 0, 0, 0);
    if (COLS == 16) b = lds16(w_addr + 8 * 64);
    uint4 xv[NG];
#pragma unroll
    for (int ng = 0; ng < NG; ++ng) {
      xv[ng] = make_uint4(0, 0, 0, 0);
      if (x_row[ng]) xv[ng] = lds16(x_addr + static_cast<uint32_t>(ng * 8) * x_stride);
    }
    const float w_s = __shfl_sync(0xffffffffu, lane_rec.scale, i & 31);
    int d[NG][4];
#pragma unroll
    for (int ng = 0; ng < NG; ++ng) {
      mma_s8_fresh(d[ng], a.x, b.x, a.y, b.y, xv[ng].x, xv[ng].y);
      mma_s8(d[ng], a.z, b.z, a.w, b.w, xv[ng].z, xv[ng].w);
    }
    if (i > 0) accumulate(d_prev, ws_prev, i - 1);
#pragma unroll
    for (int ng = 0; ng < NG; ++ng) {
#pragma unroll
      for (int e = 0; e < 4; ++e) d_prev[ng][e] = d[ng][e];
    }
    ws_prev = w_s;
    w_addr += kBlockBytes;
    x_addr += WARPS * kTile;
  }
  if (my_tiles > 0) accumulate(d_prev, ws_prev, my_tiles - 1);

  // ---- the warp sums, added in warp order ----------------------------------------------------------
  float* partial = reinterpret_cast<float*>(staged + static_cast<size_t>(warp) * warp_stage_bytes);
#pragma unroll
  for (int ng = 0; ng < NG; ++ng) {
    const int tok = ng * 8 + 2 * c;
    partial[tok * COLS + g] = acc[ng][0];
    partial[(tok + 1) * COLS + g] = acc[ng][1];
    if (COLS == 16) {
      partial[tok * COLS + g + 8] = acc[ng][2];
      partial[(tok + 1) * COLS + g + 8] = acc[ng][3];
    }
  }
  __syncthreads();
  const uint32_t epoch = kTp ? epoch_shared : 0u;
  const int32_t* meta = p.u_metadata ? p.u_metadata + static_cast<int64_t>(j) * 4 * kTile : nullptr;
  const bool has_u = kCluster && meta != nullptr && meta[0] != 0;
  const int64_t n_cols = static_cast<int64_t>(p.n_j) * kTile;
  for (int e = threadIdx.x; e < rows * COLS; e += kThreads) {
    const int row = e / COLS, col = e % COLS;
    const float* sums = reinterpret_cast<const float*>(staged) + e;  // warp 0's, the others one block further each
    float v = sums[0];
#pragma unroll
    for (int w = 1; w < WARPS; ++w) v = __fadd_rn(v, sums[w * (warp_stage_bytes / 4)]);
    if (has_u) {
      finished[row][col] = v;
    } else {
      const int64_t o = static_cast<int64_t>(row) * n_cols + static_cast<int64_t>(j) * kTile + q * COLS + col;
      if (kTp) v = sum_over_ranks(p, epoch, o, v);
      store_any(p.out, p.out_dtype, o, v);
    }
  }
  if (kCluster) {
    // Inverse output transform of a tile row: the CTAs of the cluster hold COLS columns each; CTA r
    // gathers rows r, r + kGroups, ... through distributed shared memory, one warp per row.
    cg::cluster_group cluster = cg::this_cluster();
    if (has_u) {  // the same decision in all CTAs of the cluster: they share j
      cluster.sync();
      const float* remote_lo = cluster.map_shared_rank(&finished[0][0], lane / COLS);
      const float* remote_hi = cluster.map_shared_rank(&finished[0][0], (lane + 32) / COLS);
      for (int row = q + kGroups * warp; row < rows; row += kGroups * WARPS) {
        float lo = remote_lo[row * COLS + lane % COLS];
        float hi = remote_hi[row * COLS + lane % COLS];
        inverse_u_row(lo, hi, meta, lane);
        const int64_t o = static_cast<int64_t>(row) * n_cols + static_cast<int64_t>(j) * kTile + lane;
        if (kTp) {
          lo = sum_over_ranks(p, epoch, o, lo);
          hi = sum_over_ranks(p, epoch, o + 32, hi);
        }
        store_any(p.out, p.out_dtype, o, lo);
        store_any(p.out, p.out_dtype, o + 32, hi);
      }
      cluster.sync();  // peers may still be reading this CTA's columns
    }
  }
  if (kTp) {
    // every warp has finished its exchange before the call counter may advance; the last CTA of
    // the grid advances it (the next launch starts after this one ends)
    __syncthreads();
    if (threadIdx.x == 0) {
      uint32_t* counters = reinterpret_cast<uint32_t*>(p.peers.buffer[p.tp_rank]);
      __threadfence();
      if (atomicAdd(&counters[1], 1u) == gridDim.x * gridDim.y - 1) {
        counters[1] = 0;
        counters[0] = epoch;
      }
    }
  }
}

// Shapes of the kernel: rows -> NG; 16-column CTAs of eight warps where the CTA's weights and
// activation rows fit kMaxSmem, else 8-column CTAs for at most eight rows, else the layer is left
// to the kernels that split K.
struct Shape {
  int ng;
  int cols;
  int warps;
};

constexpr int kMaxSmem = 112 * 1024;  // two CTAs per SM at least

// weights of the CTA (every slot the size of a W8 block) + the activation rows, padded by 64 bytes each
int staged_bytes(const Shape& shape, int n_k, int64_t m) {
  const int rows = static_cast<int>(m < 8 * shape.ng ? m : 8 * shape.ng);
  const int tiles_per_warp = (n_k + shape.warps - 1) / shape.warps;
  return shape.warps * static_cast<int>(warp_block_bytes(tiles_per_warp, shape.cols * kTile, 8 * shape.ng * shape.cols * 4)) +
         rows * (n_k * kTile + 64);
}

// n_j: tile rows of the layer.  Sixteen-column CTAs unless they would leave SMs without a CTA
// and eight-column CTAs (at most eight rows) are possible.
bool shape_for(int64_t m, int n_j, int n_k, Shape* shape) {
  if (m < 1 || m > 32 || n_k < 1) return false;
  const int ng = m <= 8 ? 1 : m <= 16 ? 2 : 4;
  const Shape wide = {ng, 16, 8};
  const Shape narrow = {1, 8, 8};
  const bool wide_fits = staged_bytes(wide, n_k, m) <= kMaxSmem;
  const bool narrow_fits = ng == 1 && staged_bytes(narrow, n_k, m) <= kMaxSmem;
  if (wide_fits && !(narrow_fits && static_cast<int64_t>(n_j) * (kTile / 16) < num_sms())) {
    *shape = wide;
    return true;
  }
  if (narrow_fits) {
    *shape = narrow;
    return true;
  }
  return false;
}

template <int NG, int COLS, int WARPS, bool kCluster, bool kTp, bool kQuant>
int launch_variant(const DirectParams& p, cudaStream_t stream) {
  static std::once_flag once[64];
  int device = 0;
  int rc = check_cuda(cudaGetDevice(&device), "cudaGetDevice");
  if (rc != AQ_OK) return rc;
  cudaError_t attr_status = cudaSuccess;
  std::call_once(once[device & 63], [&] {
    attr_status = cudaFuncSetAttribute(direct_decode_kernel<NG, COLS, WARPS, kCluster, kTp, kQuant>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxSmem);
  });
  rc = check_cuda(attr_status, "cudaFuncSetAttribute(direct_decode_kernel)");
  if (rc != AQ_OK) return rc;
  const Shape shape = {NG, COLS, WARPS};
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(static_cast<unsigned>(p.n_j), kTile / COLS, 1);
  config.blockDim = dim3(32 * WARPS, 1, 1);
  config.dynamicSmemBytes = static_cast<size_t>(staged_bytes(shape, p.n_k, p.m));
  config.stream = stream;
  cudaLaunchAttribute attr[2];
  int count = 0;
  if (kCluster) {
    attr[count].id = cudaLaunchAttributeClusterDimension;
    attr[count].val.clusterDim.x = 1;
    attr[count].val.clusterDim.y = kTile / COLS;
    attr[count].val.clusterDim.z = 1;
    ++count;
  }
  if (use_dependent_launch()) {
    attr[count].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[count].val.programmaticStreamSerializationAllowed = 1;
    ++count;
  }
  config.attrs = attr;
  config.numAttrs = count;
  return check_cuda(cudaLaunchKernelEx(&config, direct_decode_kernel<NG, COLS, WARPS, kCluster, kTp, kQuant>, p),
                    "direct decode launch");
}

template <int NG, int COLS, int WARPS, bool kQuant>
int launch_mode(const DirectParams& p, bool cluster, cudaStream_t stream) {
  if (p.tp_world > 1) {
    return cluster ? launch_variant<NG, COLS, WARPS, true, true, kQuant>(p, stream)
                   : launch_variant<NG, COLS, WARPS, false, true, kQuant>(p, stream);
  }
  return cluster ? launch_variant<NG, COLS, WARPS, true, false, kQuant>(p, stream)
                 : launch_variant<NG, COLS, WARPS, false, false, kQuant>(p, stream);
}

template <int NG, int COLS, int WARPS>
int launch_shape(const DirectParams& p, bool cluster, cudaStream_t stream) {
  if constexpr (NG == 1) {  // the quantizing instantiation exists for one group of rows only
    if (p.raw_x != nullptr) return launch_mode<NG, COLS, WARPS, true>(p, cluster, stream);
  }
  return launch_mode<NG, COLS, WARPS, false>(p, cluster, stream);
}

}  // namespace

// CTAs of a shape that fit one SM (shared memory, 64 Ki registers at the kernel's register count).
int ctas_per_sm(const Shape& shape, int n_k, int64_t m) {
  // 228 KiB per SM; per CTA 1 KiB for the system and the kernel's static arrays (cluster exchange, epoch)
  const int by_smem = (228 * 1024) / (staged_bytes(shape, n_k, m) + 1024 + 8 * shape.ng * shape.cols * 4 + 128);
  const int by_regs = shape.ng == 1 ? 3 : 2;  // the kernels' launch bounds
  return by_smem < by_regs ? by_smem : by_regs;
}

// The kernel pays where its CTAs (four or eight per tile row) give every SM work AND are all
// resident at once: a CTA that starts only when another one leaves runs its whole chain (records,
// weights, activations) after the dependency, in the open.  Wider layers keep the kernels that
// stream through a ring; narrower ones the kernels that split K.
bool direct_decode_supported(int64_t m, int n_j, int n_k) {
  Shape shape;
  if (!shape_for(m, n_j, n_k, &shape)) return false;
  const int64_t ctas = static_cast<int64_t>(n_j) * (kTile / shape.cols);
  // At least a CTA for every fourth SM (narrow shards of a tensor-parallel layer: a megabyte or two,
  // for which any kernel is a chain of latencies and this one has the shortest: 640 x 3072 at one row
  // 2.2 us per launch against 12 us for the stream-K kernel), and all resident.
  if (4 * ctas < num_sms() || ctas > static_cast<int64_t>(num_sms()) * ctas_per_sm(shape, n_k, m)) return false;
  // A grid that needs the SMs' shared memory to the brim to be resident is slower than the ring
  // kernel (measured: 5120 x 3072 at 8 rows, three CTAs of 74 KiB per SM, 6.1 us against 5.6 us;
  // 3072 x 8192 at one row, 8.9 us against 6.8 us): at most 200 KiB per SM.
  const int64_t per_sm = (ctas + num_sms() - 1) / num_sms();
  return per_sm * (staged_bytes(shape, n_k, m) + 2048) <= 200 * 1024;
}

// The kernel may also quantize the activations (fp16 / bf16 rows, per-token scales) where it takes
// the problem at all and the rows are few: every CTA rounds all rows, which at more rows costs
// more than the quantizer launch it saves.
bool direct_decode_quantizes(int64_t m, int n_j, int n_k) {
  return m <= kQuantRows && static_cast<int64_t>(n_j) * n_k <= quant_fusion_tiles() && direct_decode_supported(m, n_j, n_k);
}

int direct_decode_workers(int64_t m, int n_j, int n_k) {
  Shape shape;
  return shape_for(m, n_j, n_k, &shape) ? shape.warps : 0;
}

int launch_direct_decode(const LinearArgs& a, cudaStream_t stream) {
  Shape shape;
  if (!shape_for(a.m, a.n_j, a.n_k, &shape)) return fail(AQ_ERR_INVALID, "the register-staged decode kernel does not take this shape");
  DirectParams p;
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
  p.prefetch = static_cast<const uint8_t*>(a.prefetch);
  p.prefetch_bytes = a.prefetch != nullptr ? a.prefetch_bytes : 0;
  p.raw_x = a.raw_x;
  p.raw_bf16 = a.raw_dtype == AQ_BF16 ? 1 : 0;
  if (a.raw_x != nullptr && (a.m > kQuantRows || a.scale_mode != AQ_SCALE_TOKEN || (a.raw_dtype != AQ_F16 && a.raw_dtype != AQ_BF16))) {
    return fail(AQ_ERR_INVALID, "the decode kernel quantizes at most %d fp16 or bf16 rows with per-token scales", kQuantRows);
  }
  p.tp_rank = a.tp_rank;
  p.tp_world = a.peer_buffers != nullptr ? a.tp_world : 1;
  p.ar_max_count = a.ar_max_count;
  p.ar_poll_limit = peer_poll_limit();
  for (int r = 0; r < kArMaxRanks; ++r) {
    p.peers.buffer[r] = (a.peer_buffers != nullptr && r < a.tp_world) ? static_cast<uint8_t*>(a.peer_buffers[r]) : nullptr;
  }
  const bool cluster = a.u_metadata != nullptr;
  if (shape.cols == 8) return launch_shape<1, 8, 8>(p, cluster, stream);
  if (shape.ng == 1) return launch_shape<1, 16, 8>(p, cluster, stream);
  if (shape.ng == 2) return launch_shape<2, 16, 8>(p, cluster, stream);
  return launch_shape<4, 16, 8>(p, cluster, stream);
}

int take_direct_decode_status() {
  int status = 0;
  if (cudaMemcpyFromSymbol(&status, g_direct_decode_status, sizeof(int)) != cudaSuccess) return -1;
  if (status != 0) {
    const int zero = 0;
    cudaMemcpyToSymbol(g_direct_decode_status, &zero, sizeof(int));
  }
  return status;
}

}  // namespace aq
