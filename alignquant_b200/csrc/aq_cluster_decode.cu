// Decode kernel for at most 32 rows: one CTA per (tile row j, K split), split-K partial
// sums exchanged through the distributed shared memory of a thread-block cluster.
//
// This is the default small-M kernel.  It combines the two things that matter at decode
// sizes, where a whole layer is a few microseconds of HBM traffic:
//   * a byte stream that starts immediately and never stalls -- the tiles of one
//     (row, K range) are contiguous in the prepared image, so the producer warp moves
//     them with ONE bulk asynchronous copy per ring slot of eight tiles (up to 32 KiB,
//     counted on the slot's mbarrier); the first two slots are requested before the grid
//     dependency is resolved, so under programmatic dependent launch they overlap the
//     preceding kernel;
//   * tile-level parallelism -- eight consumer warps each take whole tiles (tile i of
//     the range goes to warp i % 8; weights are the 16-row operand of
//     mma.sync.m16n8k32.s8, up to eight activation rows the 8-column operand), so
//     eight tiles are in progress per CTA and, with two CTAs per SM, sixteen per SM.
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

__device__ __forceinline__ void st_volatile_v2(void* p, uint32_t a, uint32_t b) {
  asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(a), "r"(b) : "memory");
}
__device__ __forceinline__ uint2 ld_volatile_v2(const void* p) {
  uint2 v;
  asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
  return v;
}

constexpr int kGroupTiles = 8;  // tiles per ring slot
constexpr int kSlots = 2;
constexpr int kSlotBytes = kGroupTiles * kW8TileBytes;
constexpr int kTileWorkers = 8;  // tiles in progress per CTA; WPT warps share one tile (16 rows each)
constexpr int kMaxCount = 512;  // tiles of one CTA's K range
constexpr int kNumBars = 2 * kSlots;

template <int kConsumerThreads>
__device__ __forceinline__ void consumer_sync() {
  asm volatile("bar.sync 1, %0;" ::"n"(kConsumerThreads) : "memory");
}

// Shared memory: [ring kSlots x 32 KiB][slabs 8 x (8*NT) x 64 f32][tile (8*NT) x 64 f32]
//                [records kMaxCount][barriers][abort flag]
// With 16 rows (NT = 2) the slabs reuse the ring's memory once the last tile has been
// consumed (measured 4-5 % faster at M = 16: more shared memory left for the L1); with up to
// 8 rows the extra barrier that this needs costs more than it gives, so the slabs keep their
// own 16 KiB.
// For 17..32 rows two warps share every tile (WPT = 2): warp 2t takes rows 0..15 and warp
// 2t+1 rows 16..31 of tile worker t, so the weights are still streamed once.
// kTp: the epilogue also sums over the tensor-parallel ranks (a separate instantiation, so that
// the single-GPU kernel keeps its register count).
template <int NT, int WPT, bool kTp>
__global__ void __launch_bounds__(32 * (kTileWorkers * WPT + 1), WPT == 1 ? 2 : 1) cluster_decode_kernel(const Params p) {
  extern __shared__ __align__(128) uint8_t smem[];
  constexpr int kConsumerWarps = kTileWorkers * WPT;
  constexpr int kConsumerThreads = kConsumerWarps * 32;
  constexpr int kThreads = kConsumerThreads + 32;
  constexpr int kWarpRows = 8 * NT;      // rows one warp accumulates
  constexpr int kRows = kWarpRows * WPT;  // rows of the CTA
  constexpr bool kSlabsInRing = NT == 2;
  static_assert(kTileWorkers * kRows * kTile * 4 <= kSlots * kSlotBytes, "slabs must fit into the ring");
  uint8_t* ring = smem;
  float* slabs = reinterpret_cast<float*>(smem + (kSlabsInRing ? 0 : kSlots * kSlotBytes));
  float* tile = reinterpret_cast<float*>(smem + kSlots * kSlotBytes) + (kSlabsInRing ? 0 : kTileWorkers * kRows * kTile);
  TileRecord* recs = reinterpret_cast<TileRecord*>(tile + kRows * kTile);
  uint64_t* bars = reinterpret_cast<uint64_t*>(recs + kMaxCount);
  volatile uint32_t* abort_flag = reinterpret_cast<uint32_t*>(bars + kNumBars);

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

  const uint32_t bar0 = smem_u32(bars);
  auto full = [&](int s) { return bar0 + 8u * s; };
  auto empty = [&](int s) { return bar0 + 8u * (kSlots + s); };
  const uint32_t ring_addr = smem_u32(ring);

  if (threadIdx.x == 0) {
    for (int s = 0; s < kSlots; ++s) {
      mbar_init(full(s), 1);
      mbar_init(empty(s), kGroupTiles * WPT);  // every warp working on a tile arrives
    }
    *abort_flag = 0;
    mbar_init_fence();
    fence_proxy_async();
  }
  __syncthreads();

  const TileRecord* my_records = p.records + static_cast<int64_t>(j) * n_k + k_begin;
  const bool producer = warp == kConsumerWarps;  // the last warp

  // First ring fill before the grid dependency is resolved: weights are static.
  if (producer && lane < kSlots && lane < groups) {
    const int first = lane * kGroupTiles;
    const int last = (first + kGroupTiles < count ? first + kGroupTiles : count) - 1;
    const TileRecord rf = my_records[first];
    const uint32_t bytes = span_bytes(rf, my_records[last]);
    mbar_expect_tx(full(lane), bytes);
    bulk_copy(ring_addr + lane * kSlotBytes,
              p.payload + static_cast<int64_t>(rf.offset_flag & ~kW4Flag) * kW4TileBytes, bytes, full(lane));
  }
  for (int i = threadIdx.x; i < count; i += kThreads) recs[i] = my_records[i];
  grid_launch_dependents();
  grid_dependency_wait();  // activations and their scales come from the preceding kernel
  __shared__ uint32_t ar_epoch_shared;
  if (kTp && threadIdx.x == 0) {
    ar_epoch_shared = *reinterpret_cast<const volatile uint32_t*>(p.peers.buffer[p.tp_rank]) + 1;  // number of this call
  }
  __syncthreads();

  if (producer) {
    if (lane == 0) {
      for (int gi = kSlots; gi < groups; ++gi) {
        const int slot = gi % kSlots;
        if (!mbar_wait(empty(slot), ((gi / kSlots) - 1) & 1, abort_flag, &g_cluster_decode_status, 31)) break;
        const int first = gi * kGroupTiles;
        const int last = (first + kGroupTiles < count ? first + kGroupTiles : count) - 1;
        const TileRecord rf = recs[first];
        const uint32_t bytes = span_bytes(rf, recs[last]);
        mbar_expect_tx(full(slot), bytes);
        bulk_copy(ring_addr + slot * kSlotBytes,
                  p.payload + static_cast<int64_t>(rf.offset_flag & ~kW4Flag) * kW4TileBytes, bytes, full(slot));
      }
    }
    __syncwarp();
  } else {
    // Lane (g, c) = (lane/4, lane%4) holds, for column group q = 0..3, the weight vectors
    // of columns 16q+g and 16q+g+8 and the activation vector of token 8*pass+g, all for
    // k in [16c, 16c+16).  MMA results: d[0], d[1] = column 16q+g, tokens 8*pass+2c, +1;
    // d[2], d[3] = column 16q+g+8, same tokens.
    const int g = lane >> 2;
    const int c = lane & 3;
    const int64_t k_bytes = static_cast<int64_t>(n_k) * kTile;
    const uint32_t w8_off = static_cast<uint32_t>(g * 64 + ((c ^ ((g >> 1) & 3)) << 4));
    const uint32_t w4_off = static_cast<uint32_t>(g * 32 + (c >> 1) * 16);
    const int w4_shift = (c & 1) ? 0 : 4;
    float token_scale[NT][2];
    const int8_t* x_lane[NT];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      const int tok = row0 + nt * 8 + 2 * c;
      token_scale[nt][0] = (p.scale_mode == AQ_SCALE_TOKEN && tok < rows) ? p.act_scales[tok] : 0.0f;
      token_scale[nt][1] = (p.scale_mode == AQ_SCALE_TOKEN && tok + 1 < rows) ? p.act_scales[tok + 1] : 0.0f;
      x_lane[nt] = p.xq + static_cast<int64_t>(row0 + nt * 8 + g) * k_bytes + static_cast<int64_t>(k_begin) * kTile + c * 16;
    }
    auto load_x = [&](int i, uint4 (&x)[NT]) {
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        x[nt] = make_uint4(0, 0, 0, 0);
        if (row0 + nt * 8 + g < rows) x[nt] = ldg_x(x_lane[nt] + static_cast<int64_t>(i) * kTile);
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
    if (worker < count) load_x(worker, x_next);  // activation vectors are requested one tile ahead
    for (int i = worker; i < count; i += kTileWorkers) {
      const int gi = i / kGroupTiles;
      const int slot = gi % kSlots;
      const int kt = k_begin + i;
      uint4 x[NT];
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) x[nt] = x_next[nt];
      if (i + kTileWorkers < count) load_x(i + kTileWorkers, x_next);
      if (!mbar_wait(full(slot), (gi / kSlots) & 1, abort_flag, &g_cluster_decode_status, 32)) break;
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
          const float a_s = (row0 + nt * 8 < rows) ? p.act_scales[static_cast<int64_t>((row0 + nt * 8) >> 4) * n_k + kt] : 0.0f;
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
          const int tok = row0 + nt * 8 + 2 * c;
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
    // ---- combine the eight warp sums in warp order -----------------------------------------
    if (kSlabsInRing) consumer_sync<kConsumerThreads>();  // every warp has consumed its last tile: the ring becomes the slabs
    float* slab = slabs + worker * kRows * kTile;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      const int tok = row0 + nt * 8 + 2 * c;
#pragma unroll
      for (int q = 0; q < 4; ++q) {  // only the rows that exist are combined and exchanged
        if (tok < rows) {
          slab[tok * kTile + q * 16 + g] = acc[nt][q][0];
          slab[tok * kTile + q * 16 + g + 8] = acc[nt][q][2];
        }
        if (tok + 1 < rows) {
          slab[(tok + 1) * kTile + q * 16 + g] = acc[nt][q][1];
          slab[(tok + 1) * kTile + q * 16 + g + 8] = acc[nt][q][3];
        }
      }
    }
    consumer_sync<kConsumerThreads>();
    for (int e = threadIdx.x; e < rows * kTile; e += kConsumerThreads) {
      float v = slabs[e];
#pragma unroll
      for (int w = 1; w < kTileWorkers; ++w) v = __fadd_rn(v, slabs[w * kRows * kTile + e]);
      tile[e] = v;
    }
  }

  // ---- split-K exchange through cluster shared memory ------------------------------------
  // A cluster barrier costs about half a microsecond even for a single CTA: without a K split
  // (one CTA per tile row) a CTA barrier is enough, and nobody reads this CTA's tile remotely.
  if (split_k > 1) {
    cluster.sync();
  } else {
    __syncthreads();
  }
  if (!producer) {
    const int32_t* meta = p.u_metadata ? p.u_metadata + static_cast<int64_t>(j) * 4 * kTile : nullptr;
    const bool has_u = meta != nullptr && meta[0] != 0;
    const int64_t n_cols = static_cast<int64_t>(p.n_j) * kTile;
    // rank r finishes rows r, r + split_k, ...; its warps take them round robin
    if (!kTp) {
      for (int row = split + split_k * warp; row < rows; row += split_k * kConsumerWarps) {  // all consumer warps
        float lo = 0.0f, hi = 0.0f;
        for (int s = 0; s < split_k; ++s) {
          const float* remote = cluster.map_shared_rank(tile, s);
          const float a = remote[row * kTile + lane];
          const float b = remote[row * kTile + lane + 32];
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
      constexpr int kMaxOwned = (kRows + kConsumerWarps - 1) / kConsumerWarps;
      float own_lo[kMaxOwned], own_hi[kMaxOwned];
#pragma unroll
      for (int it = 0; it < kMaxOwned; ++it) {
        const int row = split + split_k * (warp + it * kConsumerWarps);
        own_lo[it] = own_hi[it] = 0.0f;
        if (row < rows) {
          float lo = 0.0f, hi = 0.0f;
          for (int s = 0; s < split_k; ++s) {
            const float* remote = cluster.map_shared_rank(tile, s);
            const float a = remote[row * kTile + lane];
            const float b = remote[row * kTile + lane + 32];
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
        const int row = split + split_k * (warp + it * kConsumerWarps);
        if (row < rows) {
          const int64_t e = static_cast<int64_t>(row) * n_cols + static_cast<int64_t>(j) * kTile + lane;
          float lo = 0.0f, hi = 0.0f;
          for (int r = 0; r < p.tp_world; ++r) {
            float a = own_lo[it], b = own_hi[it];
            if (r != p.tp_rank) {
              const uint8_t* units = p.peers.buffer[p.tp_rank] + kArHeaderBytes + (area + r * p.ar_max_count + e) * 8;
              uint2 ua = ld_volatile_v2(units);
              uint2 ub = ld_volatile_v2(units + 32 * 8);
              uint32_t polls = 0;
              while (ua.y != epoch || ub.y != epoch) {
                if (++polls >= p.ar_poll_limit) {
                  atomicCAS(&g_cluster_decode_status, 0, 40 + r);
                  break;
                }
                if (polls > 64) __nanosleep(100);
                ua = ld_volatile_v2(units);
                ub = ld_volatile_v2(units + 32 * 8);
              }
              a = __uint_as_float(ua.x);
              b = __uint_as_float(ub.x);
            }
            lo = r == 0 ? a : __fadd_rn(lo, a);
            hi = r == 0 ? b : __fadd_rn(hi, b);
          }
          store_any(p.out, p.out_dtype, e, lo);
          store_any(p.out, p.out_dtype, e + 32, hi);
        }
      }
    }
  }
  if (split_k > 1) {
    cluster.sync();  // peers may still be reading this CTA's tile
  } else if (kTp) {
    __syncthreads();  // every warp has finished its exchange before the call counter may advance
  }
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

// Kernel variants by row count: up to 8 rows <1,1>, up to 16 <2,1>, up to 32 <2,2>.
struct Variant {
  int nt;
  int wpt;
};
Variant variant_for(int64_t m) { return m <= 8 ? Variant{1, 1} : m <= 16 ? Variant{2, 1} : Variant{2, 2}; }
int variant_index(const Variant& v) { return v.wpt == 2 ? 2 : v.nt - 1; }
int variant_threads(const Variant& v) { return 32 * (kTileWorkers * v.wpt + 1); }
const void* variant_kernel(const Variant& v, bool tp = false) {
  if (tp) {
    if (v.wpt == 2) return reinterpret_cast<const void*>(cluster_decode_kernel<2, 2, true>);
    return v.nt == 1 ? reinterpret_cast<const void*>(cluster_decode_kernel<1, 1, true>)
                     : reinterpret_cast<const void*>(cluster_decode_kernel<2, 1, true>);
  }
  if (v.wpt == 2) return reinterpret_cast<const void*>(cluster_decode_kernel<2, 2, false>);
  return v.nt == 1 ? reinterpret_cast<const void*>(cluster_decode_kernel<1, 1, false>)
                   : reinterpret_cast<const void*>(cluster_decode_kernel<2, 1, false>);
}

int smem_bytes(const Variant& v) {
  const int rows = 8 * v.nt * v.wpt;
  const int slabs = v.nt == 2 ? 0 : kTileWorkers * rows * kTile * 4;  // NT = 2 keeps them in the ring
  return kSlots * kSlotBytes + slabs + rows * kTile * 4 + kMaxCount * 8 + kNumBars * 8 + 16;
}

int launch_variant(const Variant& v, const Params& p, int split_k, cudaStream_t stream) {
  static std::once_flag once[64][6];
  int device = 0;
  int rc = check_cuda(cudaGetDevice(&device), "cudaGetDevice");
  if (rc != AQ_OK) return rc;
  const bool tp = p.tp_world > 1;
  const void* kernel = variant_kernel(v, tp);
  cudaError_t attr_status = cudaSuccess;
  std::call_once(once[device & 63][variant_index(v) + (tp ? 3 : 0)], [&] {
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
  static int cache[64][3][9];  // [device][variant][split], 0 = not queried yet, -1 = failed
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
  const Variant v = variant_for(m);
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
  // own ring, and prefetching the next image on top of it was measured slower (gate_up 3072 ->
  // 16384 at one row: 9.1 us against 8.1 us per launch).
  for (int r = 0; r < kArMaxRanks; ++r) {
    p.peers.buffer[r] = (a.peer_buffers != nullptr && r < a.tp_world) ? static_cast<uint8_t*>(a.peer_buffers[r]) : nullptr;
  }
  const int split = cluster_decode_split(a.m, a.n_j, a.n_k);
  return launch_variant(variant_for(a.m), p, split, stream);
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
