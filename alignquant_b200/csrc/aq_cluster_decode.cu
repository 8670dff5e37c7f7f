// Decode kernel for at most 32 rows: one CTA per (tile row j, K split), split-K partial
// sums exchanged through the distributed shared memory of a thread-block cluster.
//
// This is the small-M kernel of the layers that do not fit a CTA's shared memory at once.  It
// combines the two things that matter at decode sizes, where a whole layer is a few
// microseconds of HBM traffic:
//   * a byte stream that starts immediately and never stalls -- the tiles of one
//     (row, K range) are contiguous in the prepared image, so ONE bulk asynchronous copy
//     moves the eight tiles of a ring slot (up to 32 KiB, counted on the slot's mbarrier);
//     the first three slots are requested before the grid dependency is resolved, so under
//     programmatic dependent launch they overlap the preceding kernel, and for the layers
//     that are split over a cluster they are the CTA's whole K range.  There is no producer
//     warp: the warp that is last to finish a slot's tiles (a counter in shared memory)
//     requests the slot's next eight.  A CTA of eight warps, not nine, also lifts the
//     compiler's register limit from 96 to 128, which the 16-row variant needs to stay
//     free of spills;
//   * tile-level parallelism -- the eight warps each take whole tiles (tile i of the range
//     goes to warp i % 8; weights are the 16-row operand of mma.sync.m16n8k32.s8, up to
//     eight activation rows the 8-column operand), so eight tiles are in progress per CTA
//     and, with two CTAs per SM, sixteen per SM.  What a warp needs to know of its tiles
//     (place in the slot, W4 flag, scale) sits in one register per lane and reaches the
//     loop by shuffle; W4 and W8 tiles take separate, branch-free instruction sequences.
// The split count is chosen so that rows x splits is at most two CTAs per SM; all CTAs
// are then co-resident and stream concurrently.
//
// Summation order (all FP32, separately rounded multiply and add as in
// alignquant/kernels/cuda/linear.cu:956-963): a warp adds its tiles in increasing k;
// the eight warp sums are added in warp order; the split sums are added in split order
// (the reference reducer's order, linear.cu:1339-1343).  No workspace, no atomics.
#include <cooperative_groups.h>

#include <mutex>

#include "aq_common.cuh"
#include "aq_ptx.cuh"
#include "aq_tile_math.cuh"

namespace cg = cooperative_groups;

namespace aq {

__device__ int g_cluster_decode_status = 0;

namespace {

struct Params {
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
  // fused sum over tensor-parallel ranks (tp_world <= 1: off)
  ArPeers peers;
  int tp_rank;
  int tp_world;
  int64_t ar_max_count;
  uint32_t ar_poll_limit;
};

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

constexpr int kGroupTiles = 8;  // tiles per ring slot
constexpr int kMaxSlots = 3;  // ring slots: 3, or 2 for the layers that are split over a cluster (see Variant)
constexpr int kModePlain = 0, kModeTp = 1, kModeDump = 2;
constexpr int kSlotBytes = kGroupTiles * kW8TileBytes;
constexpr int kTileWorkers = 8;  // tiles in progress per CTA; WPT warps share one tile (16 rows each)
constexpr int kMaxCount = 512;  // tiles of one CTA's K range
constexpr int kNumBars = kMaxSlots;  // one "slot filled" barrier per ring slot

// Counts a warp's arrival on a ring slot; release for the warp's reads of the slot, acquire for the
// one that sees the last arrival and refills it.
__device__ __forceinline__ uint32_t slot_arrive(uint32_t counter) {
  uint32_t before;
  asm volatile("atom.acq_rel.cta.shared::cta.add.u32 %0, [%1], 1;" : "=r"(before) : "r"(counter) : "memory");
  return before;
}

// The integer products of the column groups Q0 .. Q0 + QN - 1 of one staged tile with NT groups of
// eight activation rows.  `lane_base`
// is the tile's address plus this lane's offset inside a block of eight columns; the blocks of the
// four column groups and their two halves follow at fixed strides, so every read is base +
// constant.  One instantiation per tile kind: the W8 one has no selects and no shifts.
template <bool kW4, int NT, int Q0, int QN>
__device__ __forceinline__ void tile_products(const uint8_t* lane_base, int w4_shift, const uint4 (&x)[NT], int (&d)[NT][QN][4]) {
  constexpr int kHalf = kW4 ? 8 * 32 : 8 * 64;  // columns g + 8
#pragma unroll
  for (int q = 0; q < QN; ++q) {
    uint4 wa = *reinterpret_cast<const uint4*>(lane_base + (Q0 + q) * 2 * kHalf);
    uint4 wb = *reinterpret_cast<const uint4*>(lane_base + (Q0 + q) * 2 * kHalf + kHalf);
    if (kW4) {
      wa.x = (wa.x << w4_shift) & 0xf0f0f0f0u;
      wa.y = (wa.y << w4_shift) & 0xf0f0f0f0u;
      wa.z = (wa.z << w4_shift) & 0xf0f0f0f0u;
      wa.w = (wa.w << w4_shift) & 0xf0f0f0f0u;
      wb.x = (wb.x << w4_shift) & 0xf0f0f0f0u;
      wb.y = (wb.y << w4_shift) & 0xf0f0f0f0u;
      wb.z = (wb.z << w4_shift) & 0xf0f0f0f0u;
      wb.w = (wb.w << w4_shift) & 0xf0f0f0f0u;
    }
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      mma_s8_fresh(d[nt][q], wa.x, wb.x, wa.y, wb.y, x[nt].x, x[nt].y);
      mma_s8(d[nt][q], wa.z, wb.z, wa.w, wb.w, x[nt].z, x[nt].w);
    }
  }
}

// Shared memory: [ring kSlots x 32 KiB][received sums (8*NT*WPT + 7) x 64 f32][records kMaxCount][barriers]
//                [slot counters][abort flag]
// The eight warp sums ("slabs", 8 x rows x 64 f32) reuse the ring's memory once every warp has
// consumed its last tile, so that the ring can be three slots deep with two CTAs per SM: a CTA's
// first request is then up to 24 tiles, which covers the whole K range of the layers that are
// split over a cluster.
// For 17..32 rows two warps share every tile (WPT = 2): warp 2t takes rows 0..15 and warp
// 2t+1 rows 16..31 of tile worker t, so the weights are still streamed once.
// kMode: kModeTp -- the epilogue also sums over the tensor-parallel ranks; kModeDump -- the integer
// tile sums are also written out (tests).  Separate instantiations keep both out of the plain
// kernel's loop (its instructions should stay in the instruction cache) and register count.
template <int NT, int WPT, int kMode, int kSlots>
__global__ void __launch_bounds__(32 * kTileWorkers * WPT, WPT == 1 ? 2 : 1) cluster_decode_kernel(const Params p) {
  constexpr bool kTp = kMode == kModeTp;
  constexpr bool kDump = kMode == kModeDump;
  extern __shared__ __align__(128) uint8_t smem[];
  constexpr int kWarps = kTileWorkers * WPT;
  constexpr int kThreads = kWarps * 32;
  constexpr int kWarpRows = 8 * NT;      // rows one warp accumulates
  constexpr int kRows = kWarpRows * WPT;  // rows of the CTA
  constexpr int kReceivedRows = kRows + 7;  // split x ceil(rows / split) <= rows + split - 1, split <= 8
  // Rows of a slab are 68 floats apart: lane (g, c) stores to rows 2c and 2c + 1, and 2c * 68 = 8c
  // (mod 32 banks) keeps the four c of a column apart (64 would put them on one bank: 4-way conflicts,
  // measured 0.3 us per launch at 16 rows).
  constexpr int kSlabRow = kTile + 4;
  static_assert(kTileWorkers * kRows * kSlabRow * 4 <= kSlots * kSlotBytes, "slabs must fit into the ring");
  uint8_t* ring = smem;
  float* slabs = reinterpret_cast<float*>(smem);
  float* received = reinterpret_cast<float*>(smem + kSlots * kSlotBytes);  // [source CTA][owned row][64]
  TileRecord* recs = reinterpret_cast<TileRecord*>(received + kReceivedRows * kTile);
  uint64_t* bars = reinterpret_cast<uint64_t*>(recs + kMaxCount);
  uint32_t* consumed = reinterpret_cast<uint32_t*>(bars + kNumBars);  // warps that are done with the slot's current tiles
  volatile uint32_t* abort_flag = consumed + kMaxSlots;

  cg::cluster_group cluster = cg::this_cluster();
  const int split_k = static_cast<int>(cluster.num_blocks());
  const int split = static_cast<int>(cluster.block_rank());
  const int j = blockIdx.x;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int worker = warp / WPT;                  // which of the eight tiles in progress
  const int row0 = (warp % WPT) * kWarpRows;      // first row this warp accumulates
  const int n_k = p.n_k;
  const int k_begin = static_cast<int>(static_cast<int64_t>(n_k) * split / split_k);
  const int k_end = static_cast<int>(static_cast<int64_t>(n_k) * (split + 1) / split_k);
  const int count = k_end - k_begin;
  const int groups = (count + kGroupTiles - 1) / kGroupTiles;
  const int rows = p.m < kRows ? static_cast<int>(p.m) : kRows;
  const int owned_rows = (rows + split_k - 1) / split_k;  // rows a CTA of the cluster finishes, at most

  const uint32_t bar0 = smem_u32(bars);
  auto full = [&](int s) { return bar0 + 8u * s; };
  const uint32_t ring_addr = smem_u32(ring);

  if (threadIdx.x == 0) {
    for (int s = 0; s < kSlots; ++s) {
      mbar_init(full(s), 1);
      consumed[s] = 0;
    }
    *abort_flag = 0;
    mbar_init_fence();
    fence_proxy_async();
  }
  __syncthreads();

  const TileRecord* my_records = p.records + static_cast<int64_t>(j) * n_k + k_begin;

  // First ring fill before the grid dependency is resolved: weights are static.
  if (warp == 0 && lane < kSlots && lane < groups) {
    const int first = lane * kGroupTiles;
    const int last = (first + kGroupTiles < count ? first + kGroupTiles : count) - 1;
    const TileRecord rf = my_records[first];
    const uint32_t bytes = span_bytes(rf, my_records[last]);
    mbar_expect_tx(full(lane), bytes);
    bulk_copy(ring_addr + lane * kSlotBytes,
              p.payload + static_cast<int64_t>(rf.offset_flag & ~kW4Flag) * kW4TileBytes, bytes, full(lane));
  }
  if (groups > kSlots) {  // only the later fills read the records from shared memory
    for (int i = threadIdx.x; i < count; i += kThreads) recs[i] = my_records[i];
  }
  // A tile worker takes tile t of the CTA's range from every group of eight: tile worker + 8 t,
  // which lies in ring slot t % kSlots.  Lane l keeps what the loop needs of the warp's tile l
  // (of tile 32 b + l in the b-th block of 32): its byte offset inside the slot, the W4 flag and
  // the scale, so that the loop gets them with two shuffles instead of shared-memory reads and
  // address arithmetic.  All of this, and every kernel parameter the loop uses, is read here,
  // before the dependency: afterwards each first read would be a round trip of its own.
  const int my_tiles = worker < count ? (count - worker + kTileWorkers - 1) / kTileWorkers : 0;
  uint32_t lane_off = 0;
  float lane_scale = 0.0f;
  auto load_lane_records = [&](int t0) {
    lane_off = 0;
    lane_scale = 0.0f;
    const int t = t0 + lane;
    if (t < my_tiles) {
      const TileRecord r = my_records[worker + kTileWorkers * t];
      const TileRecord r0 = my_records[kGroupTiles * t];  // first tile of the group, which starts the slot
      lane_off = (((r.offset_flag & ~kW4Flag) - (r0.offset_flag & ~kW4Flag)) * kW4TileBytes) | (r.offset_flag & kW4Flag);
      lane_scale = r.scale;
    }
  };
  load_lane_records(0);
  const int g = lane >> 2;
  const int c = lane & 3;
  const bool token_mode = p.scale_mode == AQ_SCALE_TOKEN;
  const float* const scale_global = p.act_scales;
  int32_t* const dump_global = kDump ? p.acc_dump : nullptr;
  const int64_t k_bytes = static_cast<int64_t>(n_k) * kTile;
  const int8_t* x_lane[NT];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    x_lane[nt] = p.xq + static_cast<int64_t>(row0 + nt * 8 + g) * k_bytes + static_cast<int64_t>(k_begin + worker) * kTile + c * 16;
  }
  grid_launch_dependents();
  grid_dependency_wait();  // activations and their scales come from the preceding kernel
  __shared__ uint32_t ar_epoch_shared;
  if (kTp && threadIdx.x == 0) {
    ar_epoch_shared = *reinterpret_cast<const volatile uint32_t*>(p.peers.buffer[p.tp_rank]) + 1;  // number of this call
  }
  __syncthreads();

  {
    // Lane (g, c) = (lane/4, lane%4) holds, for column group q = 0..3, the weight vectors
    // of columns 16q+g and 16q+g+8 and the activation vector of token 8*pass+g, all for
    // k in [16c, 16c+16).  MMA results: d[0], d[1] = column 16q+g, tokens 8*pass+2c, +1;
    // d[2], d[3] = column 16q+g+8, same tokens.
    const uint32_t w8_off = static_cast<uint32_t>(g * 64 + ((c ^ ((g >> 1) & 3)) << 4));
    const uint32_t w4_off = static_cast<uint32_t>(g * 32 + (c >> 1) * 16);
    const int w4_shift = (c & 1) ? 0 : 4;
    float token_scale[NT][2];
    bool x_row[NT];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      const int tok = row0 + nt * 8 + 2 * c;
      token_scale[nt][0] = (token_mode && tok < rows) ? scale_global[tok] : 0.0f;
      token_scale[nt][1] = (token_mode && tok + 1 < rows) ? scale_global[tok + 1] : 0.0f;
      x_row[nt] = row0 + nt * 8 + g < rows;
    }
    auto load_x = [&](uint4 (&x)[NT]) {  // the activation vectors of the warp's next tile
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        x[nt] = make_uint4(0, 0, 0, 0);
        if (x_row[nt]) x[nt] = ldg_x(x_lane[nt]);
        x_lane[nt] += kTileWorkers * kTile;
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
    uint4 x_next[NT];
    if (my_tiles > 0) load_x(x_next);  // activation vectors are requested one tile ahead
    int slot = 0;
    uint32_t parity = 0;
    for (int t = 0; t < my_tiles; ++t) {
      if (t != 0 && (t & 31) == 0) load_lane_records(t);  // very long K ranges: the next block of records
      uint4 x[NT];
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) x[nt] = x_next[nt];
      if (t + 1 < my_tiles) load_x(x_next);
      // the same decision in all lanes: the shuffles below need the whole warp
      if (!__all_sync(0xffffffffu, mbar_wait(full(slot), parity, abort_flag, &g_cluster_decode_status, 32))) break;
      const uint32_t of = __shfl_sync(0xffffffffu, lane_off, t & 31);
      const float w_s = __shfl_sync(0xffffffffu, lane_scale, t & 31);
      const bool is_w4 = (of & kW4Flag) != 0;
      const uint8_t* staged = ring + slot * kSlotBytes + (of & ~kW4Flag);
      const int kt = k_begin + worker + kTileWorkers * t;
      float s0[NT], s1[NT];
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        if (token_mode) {
          s0[nt] = __fmul_rn(token_scale[nt][0], w_s);
          s1[nt] = __fmul_rn(token_scale[nt][1], w_s);
        } else {
          // tokens 8*nt .. 8*nt+7 share the scale of their 16-row group
          const float a_s = (row0 + nt * 8 < rows) ? scale_global[static_cast<int64_t>((row0 + nt * 8) >> 4) * n_k + kt] : 0.0f;
          s0[nt] = s1[nt] = __fmul_rn(a_s, w_s);
        }
      }
      // Sixteen rows: two column groups at a time, so that only half of the integer sums are live.
      constexpr int QN = NT == 1 ? 4 : 2;
#pragma unroll
      for (int q0 = 0; q0 < 4; q0 += QN) {
        int d[NT][QN][4];
        if (is_w4) {
          if (q0 == 0) tile_products<true, NT, 0, QN>(staged + w4_off, w4_shift, x, d);
          else tile_products<true, NT, 4 - QN, QN>(staged + w4_off, w4_shift, x, d);
        } else {
          if (q0 == 0) tile_products<false, NT, 0, QN>(staged + w8_off, 0, x, d);
          else tile_products<false, NT, 4 - QN, QN>(staged + w8_off, 0, x, d);
        }
        if (q0 + QN == 4) {
          // Every lane's operands have been consumed by the warp-wide MMAs: this tile is done.  The
          // warp that sees all others done with the group refills the slot with the group kSlots later.
          __syncwarp();
          if (lane == 0 && t + kSlots < groups && slot_arrive(smem_u32(consumed + slot)) == kGroupTiles * WPT - 1) {
            consumed[slot] = 0;  // the next arrivals come after the new tiles have landed
            const int first = (t + kSlots) * kGroupTiles;
            const int last = (first + kGroupTiles < count ? first + kGroupTiles : count) - 1;
            const TileRecord rf = recs[first];
            const uint32_t bytes = span_bytes(rf, recs[last]);
            mbar_expect_tx(full(slot), bytes);
            bulk_copy(ring_addr + slot * kSlotBytes,
                      p.payload + static_cast<int64_t>(rf.offset_flag & ~kW4Flag) * kW4TileBytes, bytes, full(slot));
          }
        }
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
          for (int q = 0; q < QN; ++q) {
            acc[nt][q0 + q][0] = __fadd_rn(acc[nt][q0 + q][0], __fmul_rn(static_cast<float>(d[nt][q][0]), s0[nt]));
            acc[nt][q0 + q][1] = __fadd_rn(acc[nt][q0 + q][1], __fmul_rn(static_cast<float>(d[nt][q][1]), s1[nt]));
            acc[nt][q0 + q][2] = __fadd_rn(acc[nt][q0 + q][2], __fmul_rn(static_cast<float>(d[nt][q][2]), s0[nt]));
            acc[nt][q0 + q][3] = __fadd_rn(acc[nt][q0 + q][3], __fmul_rn(static_cast<float>(d[nt][q][3]), s1[nt]));
          }
          if (kDump) {
            const int shift = is_w4 ? 4 : 0;
            const int tok = row0 + nt * 8 + 2 * c;
#pragma unroll
            for (int q = 0; q < QN; ++q) {
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const int tk = tok + (e & 1);
                const int col = (q0 + q) * 16 + g + ((e & 2) ? 8 : 0);
                if (tk < rows) {
                  dump_global[((static_cast<int64_t>(tk) * p.n_j + j) * n_k + kt) * kTile + col] = d[nt][q][e] >> shift;
                }
              }
            }
          }
        }
      }
      if (++slot == kSlots) {
        slot = 0;
        parity ^= 1u;
      }
    }
    // ---- combine the eight warp sums in warp order -----------------------------------------
    __syncthreads();  // every warp has consumed its last tile: the ring becomes the slabs
    float* slab = slabs + worker * kRows * kSlabRow;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      const int tok = row0 + nt * 8 + 2 * c;
#pragma unroll
      for (int q = 0; q < 4; ++q) {  // only the rows that exist are combined and exchanged
        if (tok < rows) {
          slab[tok * kSlabRow + q * 16 + g] = acc[nt][q][0];
          slab[tok * kSlabRow + q * 16 + g + 8] = acc[nt][q][2];
        }
        if (tok + 1 < rows) {
          slab[(tok + 1) * kSlabRow + q * 16 + g] = acc[nt][q][1];
          slab[(tok + 1) * kSlabRow + q * 16 + g + 8] = acc[nt][q][3];
        }
      }
    }
    __syncthreads();
    // The CTA's sum of row r goes straight to the CTA that finishes the row (r % split_k), into
    // the place of this CTA's K range there: after ONE cluster barrier every CTA adds what it
    // received, in its own shared memory, and nobody has to stay for a peer that still reads.
    for (int e = threadIdx.x; e < rows * kTile; e += kThreads) {
      const int row = e / kTile, col = e % kTile;
      const float* sums = slabs + row * kSlabRow + col;
      float v = sums[0];
#pragma unroll
      for (int w = 1; w < kTileWorkers; ++w) v = __fadd_rn(v, sums[w * kRows * kSlabRow]);
      const int owner = row % split_k, place = row / split_k;
      float* target = split_k > 1 ? cluster.map_shared_rank(received, owner) : received;
      target[(split * owned_rows + place) * kTile + col] = v;
    }
  }

  // ---- split-K sums: every CTA adds what the cluster sent it -------------------------------
  // A cluster barrier costs about half a microsecond even for a single CTA: without a K split
  // (one CTA per tile row) a CTA barrier is enough.
  if (split_k > 1) {
    cluster.sync();
  } else {
    __syncthreads();
  }
  {
    const int32_t* meta = p.u_metadata ? p.u_metadata + static_cast<int64_t>(j) * 4 * kTile : nullptr;
    const bool has_u = meta != nullptr && meta[0] != 0;
    const int64_t n_cols = static_cast<int64_t>(p.n_j) * kTile;
    // rank r finishes rows r, r + split_k, ...; its warps take them round robin
    if (!kTp) {
      for (int row = split + split_k * warp; row < rows; row += split_k * kWarps) {  // all consumer warps
        float lo = 0.0f, hi = 0.0f;
        for (int s = 0; s < split_k; ++s) {
          const float* from = received + (s * owned_rows + row / split_k) * kTile;
          const float a = from[lane];
          const float b = from[lane + 32];
          lo = (s == 0) ? a : __fadd_rn(lo, a);
          hi = (s == 0) ? b : __fadd_rn(hi, b);
        }
        if (has_u) inverse_u_row(lo, hi, meta, lane);
        const int64_t o = static_cast<int64_t>(row) * n_cols + static_cast<int64_t>(j) * kTile + lane;
        store_any(p.out, p.out_dtype, o, lo);
        store_any(p.out, p.out_dtype, o + 32, hi);
      }
    } else {
      // Row-parallel layer: the finished values of this rank go, each paired with the call number
      // in one 8-byte unit, into the receive area of every peer (plain NVLink stores); the same
      // lane then polls the peers' units of the same positions in its own receive area (bounded)
      // and adds the ranks' values in rank order -- the protocol of aq_allreduce.cu, without a
      // second launch.
      const uint32_t epoch = ar_epoch_shared;
      const int64_t area = (static_cast<int64_t>(epoch & 1u) * p.tp_world) * p.ar_max_count;  // values
      constexpr int kMaxOwned = (kRows + kWarps - 1) / kWarps;
      float own_lo[kMaxOwned], own_hi[kMaxOwned];
#pragma unroll
      for (int it = 0; it < kMaxOwned; ++it) {
        const int row = split + split_k * (warp + it * kWarps);
        own_lo[it] = own_hi[it] = 0.0f;
        if (row < rows) {
          float lo = 0.0f, hi = 0.0f;
          for (int s = 0; s < split_k; ++s) {
            const float* from = received + (s * owned_rows + row / split_k) * kTile;
            const float a = from[lane];
            const float b = from[lane + 32];
            lo = (s == 0) ? a : __fadd_rn(lo, a);
            hi = (s == 0) ? b : __fadd_rn(hi, b);
          }
          if (has_u) inverse_u_row(lo, hi, meta, lane);
          own_lo[it] = lo;
          own_hi[it] = hi;
          const int64_t e = static_cast<int64_t>(row) * n_cols + static_cast<int64_t>(j) * kTile + lane;
          for (int step = 1; step < p.tp_world; ++step) {
            const int peer = (p.tp_rank + step) % p.tp_world;
            uint8_t* units = p.peers.buffer[peer] + kArHeaderBytes + (area + p.tp_rank * p.ar_max_count + e) * 8;
            st_volatile_v2(units, __float_as_uint(lo), epoch);
            st_volatile_v2(units + 32 * 8, __float_as_uint(hi), epoch);
          }
        }
      }
#pragma unroll
      for (int it = 0; it < kMaxOwned; ++it) {
        const int row = split + split_k * (warp + it * kWarps);
        if (row < rows) {
          const int64_t e = static_cast<int64_t>(row) * n_cols + static_cast<int64_t>(j) * kTile + lane;
          // the peers' units are requested together and re-requested only where the tag is still
          // old: one L2 round trip for all ranks that have delivered, not one per rank
          const uint8_t* const mine = p.peers.buffer[p.tp_rank] + kArHeaderBytes + (area + e) * 8;
          const int64_t rank_stride = p.ar_max_count * 8;
          uint2 ua[kArMaxRanks], ub[kArMaxRanks];
#pragma unroll
          for (int r = 0; r < kArMaxRanks; ++r) {
            ua[r] = ub[r] = make_uint2(0u, epoch);
            if (r < p.tp_world && r != p.tp_rank) {
              ua[r] = ld_volatile_v2(mine + r * rank_stride);
              ub[r] = ld_volatile_v2(mine + r * rank_stride + 32 * 8);
            }
          }
          for (uint32_t polls = 0;;) {
            bool complete = true;
#pragma unroll
            for (int r = 0; r < kArMaxRanks; ++r) {
              if (ua[r].y != epoch || ub[r].y != epoch) {
                complete = false;
                ua[r] = ld_volatile_v2(mine + r * rank_stride);
                ub[r] = ld_volatile_v2(mine + r * rank_stride + 32 * 8);
              }
            }
            if (complete) break;
            if (++polls >= p.ar_poll_limit) {
              int late = 0;
#pragma unroll
              for (int r = 0; r < kArMaxRanks; ++r) late = ((ua[r].y != epoch || ub[r].y != epoch) && late == 0) ? 40 + r : late;
              if (late != 0) atomicCAS(&g_cluster_decode_status, 0, late);
              break;
            }
            if (polls > 64) __nanosleep(100);
          }
          float lo = 0.0f, hi = 0.0f;
#pragma unroll
          for (int r = 0; r < kArMaxRanks; ++r) {
            if (r < p.tp_world) {
              const float a = r == p.tp_rank ? own_lo[it] : __uint_as_float(ua[r].x);
              const float b = r == p.tp_rank ? own_hi[it] : __uint_as_float(ub[r].x);
              lo = r == 0 ? a : __fadd_rn(lo, a);
              hi = r == 0 ? b : __fadd_rn(hi, b);
            }
          }
          store_any(p.out, p.out_dtype, e, lo);
          store_any(p.out, p.out_dtype, e + 32, hi);
        }
      }
    }
  }
  if (kTp) __syncthreads();  // every warp has finished its exchange before the call counter may advance
  if (kTp && threadIdx.x == 0) {
    // the last CTA of the grid advances the call counter (the next launch starts after this one ends)
    uint32_t* counters = reinterpret_cast<uint32_t*>(p.peers.buffer[p.tp_rank]);
    __threadfence();
    if (atomicAdd(&counters[1], 1u) == gridDim.x * gridDim.y - 1) {
      counters[1] = 0;
      counters[0] = ar_epoch_shared;
    }
  }
}

// Kernel variants by row count: up to 8 rows <1,1>, up to 16 <2,1>, up to 32 <2,2>; and by ring
// depth: layers that are split over a cluster have short K ranges per CTA (their first two slots
// are most or all of it), so they run with two slots and leave 32 KiB per CTA to the CTAs of the
// next launch; unsplit layers stream a whole tile row through three.
struct Variant {
  int nt;
  int wpt;
  int slots;
};
Variant variant_for(int64_t m, int split) {
  const int slots = (split > 1 && m <= 16) ? 2 : 3;  // the 32-row variant's warp sums need the third slot
  return m <= 8 ? Variant{1, 1, slots} : m <= 16 ? Variant{2, 1, slots} : Variant{2, 2, 3};
}
int variant_index(const Variant& v) { return (v.wpt == 2 ? 2 : v.nt - 1) + (v.slots == 2 ? 3 : 0); }  // 0..4
constexpr int kVariants = 5;
int variant_threads(const Variant& v) { return 32 * kTileWorkers * v.wpt; }
template <int kMode>
const void* variant_kernel_of(const Variant& v) {
  if (v.wpt == 2) return reinterpret_cast<const void*>(cluster_decode_kernel<2, 2, kMode, 3>);
  if (v.slots == 2) {
    return v.nt == 1 ? reinterpret_cast<const void*>(cluster_decode_kernel<1, 1, kMode, 2>)
                     : reinterpret_cast<const void*>(cluster_decode_kernel<2, 1, kMode, 2>);
  }
  return v.nt == 1 ? reinterpret_cast<const void*>(cluster_decode_kernel<1, 1, kMode, 3>)
                   : reinterpret_cast<const void*>(cluster_decode_kernel<2, 1, kMode, 3>);
}
const void* variant_kernel(const Variant& v, int mode = kModePlain) {
  return mode == kModeTp ? variant_kernel_of<kModeTp>(v) : mode == kModeDump ? variant_kernel_of<kModeDump>(v)
                                                                              : variant_kernel_of<kModePlain>(v);
}

int smem_bytes(const Variant& v) {
  const int rows = 8 * v.nt * v.wpt;  // the slabs live in the ring
  return v.slots * kSlotBytes + (rows + 7) * kTile * 4 + kMaxCount * 8 + kNumBars * 8 + kMaxSlots * 4 + 16;
}

int launch_variant(const Variant& v, const Params& p, int split_k, cudaStream_t stream) {
  static std::once_flag once[64][3 * kVariants];
  int device = 0;
  int rc = check_cuda(cudaGetDevice(&device), "cudaGetDevice");
  if (rc != AQ_OK) return rc;
  const int mode = p.tp_world > 1 ? kModeTp : p.acc_dump != nullptr ? kModeDump : kModePlain;
  const void* kernel = variant_kernel(v, mode);
  cudaError_t attr_status = cudaSuccess;
  std::call_once(once[device & 63][variant_index(v) + kVariants * mode], [&] {
    attr_status = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes(v));
  });
  rc = check_cuda(attr_status, "cudaFuncSetAttribute(cluster_decode_kernel)");
  if (rc != AQ_OK) return rc;
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(static_cast<unsigned>(p.n_j), static_cast<unsigned>(split_k), 1);
  config.blockDim = dim3(static_cast<unsigned>(variant_threads(v)), 1, 1);
  config.dynamicSmemBytes = static_cast<size_t>(smem_bytes(v));
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
  Params params = p;
  void* args[] = {&params};
  return check_cuda(cudaLaunchKernelExC(&config, kernel, args), "cluster decode launch");
}

}  // namespace

namespace {

// How many clusters of `split` CTAs of a variant can be resident at once on the current
// device (0 when the query fails); cached per device.
int max_active_clusters(const Variant& v, int split) {
  static std::mutex mutex;
  static int cache[64][kVariants][9];  // [device][variant][split], 0 = not queried yet, -1 = failed
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return 0;
  std::lock_guard<std::mutex> lock(mutex);
  int& slot = cache[device][variant_index(v)][split];
  if (slot == 0) {
    const void* kernel = variant_kernel(v);
    cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes(v));
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(1, static_cast<unsigned>(split), 1);
    config.blockDim = dim3(static_cast<unsigned>(variant_threads(v)), 1, 1);
    config.dynamicSmemBytes = static_cast<size_t>(smem_bytes(v));
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = static_cast<unsigned>(split);
    attr[0].val.clusterDim.z = 1;
    config.attrs = attr;
    config.numAttrs = 1;
    int clusters = 0;
    const cudaError_t status = cudaOccupancyMaxActiveClusters(&clusters, kernel, &config);
    if (status != cudaSuccess) (void)cudaGetLastError();
    slot = (status == cudaSuccess && clusters > 0) ? clusters : -1;
  }
  return slot > 0 ? slot : 0;
}

}  // namespace

// Largest split (cluster size, at most 8) for which the grid is at most two CTAs per SM (one
// for the 32-row variant, whose CTAs fill an SM) and all n_j clusters are resident at once, so
// that every CTA streams from the start; never shorter than one tile per CTA and never longer
// than the record buffer.
int cluster_decode_split(int64_t m, int n_j, int n_k) {
  const Variant v = variant_for(m, 2);  // what a split layer runs
  static int sm_count[64] = {0};
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) device = 0;
  if (sm_count[device] == 0) {
    int count = 0;
    if (cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || count <= 0) count = 148;
    sm_count[device] = count;
  }
  const int64_t cta_limit = (v.wpt == 2 ? 1LL : 2LL) * sm_count[device];
  int split = 1;
  for (int s = 2; s <= 8 && s <= n_k; ++s) {
    if (static_cast<int64_t>(n_j) * s <= cta_limit && max_active_clusters(v, s) >= n_j) split = s;
  }
  while (split < 8 && (n_k + split - 1) / split > kMaxCount) ++split;
  return split;
}

bool cluster_decode_supported(int n_j, int n_k) { return (n_k + 7) / 8 <= kMaxCount && n_j > 0; }

int launch_cluster_decode(const LinearArgs& a, cudaStream_t stream) {
  Params p;
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
  p.tp_rank = a.tp_rank;
  p.tp_world = a.peer_buffers != nullptr ? a.tp_world : 1;
  p.ar_max_count = a.ar_max_count;
  p.ar_poll_limit = peer_poll_limit();
  // The look-ahead hint of aq_linear_ahead is not used here: this kernel keeps HBM busy with its
  // own ring.  Prefetching the next image was measured both at the start of the kernel (slower:
  // 9.1 us against 8.1 us per launch of the 3072 -> 16384 layer at one row) and at the end of the
  // tile loop (no gain for the kernel that follows).
  for (int r = 0; r < kArMaxRanks; ++r) {
    p.peers.buffer[r] = (a.peer_buffers != nullptr && r < a.tp_world) ? static_cast<uint8_t*>(a.peer_buffers[r]) : nullptr;
  }
  const int split = cluster_decode_split(a.m, a.n_j, a.n_k);
  return launch_variant(variant_for(a.m, split), p, split, stream);
}

int take_cluster_decode_status() {
  int status = 0;
  if (cudaMemcpyFromSymbol(&status, g_cluster_decode_status, sizeof(int)) != cudaSuccess) return -1;
  if (status != 0) {
    const int zero = 0;
    cudaMemcpyToSymbol(g_cluster_decode_status, &zero, sizeof(int));
  }
  return status;
}

}  // namespace aq
