// Sum of the partial outputs of a row-parallel projection over the ranks of one node,
// through peer memory (NVLink / NVSwitch), for the small messages of decode.  The reference has
// no counterpart: it runs on one GPU and contains no collective; this replaces the
// dist.all_reduce that tensor parallelism needs after a row-parallel projection.
//
// Every rank owns one "exchange buffer" that all peers have mapped:
//   [ call counter, CTA counter | pad to 1024 B | recv[2][world][max_count] x {float value, uint32 epoch} ]
// One launch per rank and all-reduce, up to kBlocks CTAs (one per 1024 values), each thread
// owning groups of four values:
//   1. epoch = call counter + 1 (the number of this all-reduce, the same in every CTA and on
//      every rank; it lives on the device, so a captured launch can be replayed; the last CTA
//      to finish stores it back), parity = epoch & 1;
//   2. push: every value travels together with the epoch in one 8-byte unit (two units per
//      16-byte store) into recv[parity][rank] of every peer over NVLink.  There is no separate
//      flag and no fence: a unit whose tag equals the epoch carries this all-reduce's value,
//      because an aligned 8-byte unit is never torn;
//   3. the same thread polls the units of its groups in its own recv[parity][peer] until
//      their tags match (bounded: on a time-out it records the peer in a status word and goes
//      on, so a missing peer turns into an error code instead of a hang) and adds the values in
//      rank order 0..world-1 (its own from the partial), which gives every rank the same bits.
// Two recv halves are enough: a rank can only reach all-reduce e+2 after it has received
// every peer's e+1, which a peer sends after it has finished reading e.  The tag wraps after
// 2^32 calls per buffer.
// Only plain peer stores and local loads are used: no multicast objects, no multimem.
#include "aq_common.cuh"

namespace aq {

__device__ int g_allreduce_status = 0;

namespace {

constexpr int kBlocks = 16;
constexpr int kMaxRanks = kArMaxRanks;
constexpr int kThreads = 256;
constexpr int kHeaderBytes = kArHeaderBytes;
static_assert(kBlocks * 4 <= kHeaderBytes, "header too small");

using Peers = ArPeers;

// Two exchange units {value, call number} per 16-byte access, as a vector of two 64-bit scalars:
// each unit is single-copy atomic, so a reader never sees a new tag with an old value.
__device__ __forceinline__ void st_volatile_v4(uint4* p, const uint4& v) {
  const uint64_t a = static_cast<uint64_t>(v.x) | (static_cast<uint64_t>(v.y) << 32);
  const uint64_t b = static_cast<uint64_t>(v.z) | (static_cast<uint64_t>(v.w) << 32);
  asm volatile("st.volatile.global.v2.u64 [%0], {%1, %2};" ::"l"(p), "l"(a), "l"(b) : "memory");
}
__device__ __forceinline__ uint4 ld_volatile_v4(const uint4* p) {
  uint64_t a, b;
  asm volatile("ld.volatile.global.v2.u64 {%0, %1}, [%2];" : "=l"(a), "=l"(b) : "l"(p) : "memory");
  return make_uint4(static_cast<uint32_t>(a), static_cast<uint32_t>(a >> 32), static_cast<uint32_t>(b), static_cast<uint32_t>(b >> 32));
}

__global__ void __launch_bounds__(kThreads) allreduce_push_kernel(const float* __restrict__ partial,
                                                                  float* __restrict__ out, int64_t count,
                                                                  int rank, int world, int64_t max_count,
                                                                  uint32_t poll_limit, const Peers peers) {
  __shared__ uint32_t epoch_shared;
  const int b = blockIdx.x;
  const int blocks = static_cast<int>(gridDim.x);
  uint8_t* mine = peers.buffer[rank];
  uint32_t* counters = reinterpret_cast<uint32_t*>(mine);
  if (threadIdx.x == 0) epoch_shared = counters[0] + 1;
  __syncthreads();
  const uint32_t epoch = epoch_shared;
  // recv[parity][r] starts at uint4 index (parity * world + r) * max_count / 2 (8 bytes per value)
  const int64_t half = static_cast<int64_t>(epoch & 1u) * world;
  const int64_t rank_stride = max_count >> 1;

  // groups of four values; group i of a rank's area occupies uint4 2i and 2i+1
  const int64_t groups = count >> 2;
  const int64_t per_block = (groups + blocks - 1) / blocks;
  const int64_t g_begin = b * per_block;
  const int64_t g_end = g_begin + per_block < groups ? g_begin + per_block : groups;

  const float4* src = reinterpret_cast<const float4*>(partial);
  for (int64_t i = g_begin + threadIdx.x; i < g_end; i += kThreads) {
    const float4 v = src[i];
    const uint4 lo = make_uint4(__float_as_uint(v.x), epoch, __float_as_uint(v.y), epoch);
    const uint4 hi = make_uint4(__float_as_uint(v.z), epoch, __float_as_uint(v.w), epoch);
    for (int step = 1; step < world; ++step) {
      const int peer = (rank + step) % world;  // every rank starts with a different peer
      uint4* dst = reinterpret_cast<uint4*>(peers.buffer[peer] + kHeaderBytes) + (half + rank) * rank_stride + 2 * i;
      st_volatile_v4(dst, lo);
      st_volatile_v4(dst + 1, hi);
    }
  }

  const uint4* recv = reinterpret_cast<const uint4*>(mine + kHeaderBytes) + half * rank_stride;
  float4* dst = reinterpret_cast<float4*>(out);
  for (int64_t i = g_begin + threadIdx.x; i < g_end; i += kThreads) {
    const float4 own = src[i];
    // the peers' units are requested together and re-requested only where a tag is still old
    const uint4* const units = recv + 2 * i;
    uint4 lo[kMaxRanks], hi[kMaxRanks];
#pragma unroll
    for (int r = 0; r < kMaxRanks; ++r) {
      lo[r] = hi[r] = make_uint4(0u, epoch, 0u, epoch);
      if (r < world && r != rank) {
        lo[r] = ld_volatile_v4(units + r * rank_stride);
        hi[r] = ld_volatile_v4(units + r * rank_stride + 1);
      }
    }
    for (uint32_t polls = 0;;) {
      bool complete = true;
#pragma unroll
      for (int r = 0; r < kMaxRanks; ++r) {
        if (lo[r].y != epoch || lo[r].w != epoch || hi[r].y != epoch || hi[r].w != epoch) {
          complete = false;
          lo[r] = ld_volatile_v4(units + r * rank_stride);
          hi[r] = ld_volatile_v4(units + r * rank_stride + 1);
        }
      }
      if (complete) break;
      if (++polls >= poll_limit) {
        int late = 0;
#pragma unroll
        for (int r = 0; r < kMaxRanks; ++r) {
          const bool old = lo[r].y != epoch || lo[r].w != epoch || hi[r].y != epoch || hi[r].w != epoch;
          late = (old && late == 0) ? 1 + r : late;
        }
        if (late != 0) atomicCAS(&g_allreduce_status, 0, late);
        break;
      }
      if (polls > 64) __nanosleep(100);
    }
    float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
    for (int r = 0; r < kMaxRanks; ++r) {
      if (r < world) {
        const float4 v = r == rank ? own
                                   : make_float4(__uint_as_float(lo[r].x), __uint_as_float(lo[r].z), __uint_as_float(hi[r].x),
                                                 __uint_as_float(hi[r].z));
        if (r == 0) {
          acc = v;
        } else {
          acc.x = __fadd_rn(acc.x, v.x);
          acc.y = __fadd_rn(acc.y, v.y);
          acc.z = __fadd_rn(acc.z, v.z);
          acc.w = __fadd_rn(acc.w, v.w);
        }
      }
    }
    dst[i] = acc;
  }
  // the last CTA to finish advances the call counter (the next launch starts after this one ends)
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(&counters[1], 1u) == static_cast<uint32_t>(blocks - 1)) {
      counters[1] = 0;
      counters[0] = epoch;
    }
  }
}

}  // namespace

int64_t allreduce_buffer_bytes(int world, int64_t max_count) {
  return kHeaderBytes + 2 * static_cast<int64_t>(world) * max_count * 8;  // 8 bytes per value: {value, epoch}
}

int allreduce_max_ranks() { return kMaxRanks; }

int launch_allreduce(const float* partial, float* out, int64_t count, int rank, int world, void* const* peer_buffers,
                     int64_t max_count, cudaStream_t stream) {
  Peers peers;
  for (int r = 0; r < kMaxRanks; ++r) peers.buffer[r] = r < world ? static_cast<uint8_t*>(peer_buffers[r]) : nullptr;
  int64_t blocks = (count / 4 + kThreads - 1) / kThreads;  // the same on every rank: count is
  if (blocks > kBlocks) blocks = kBlocks;
  if (blocks < 1) blocks = 1;
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(static_cast<unsigned>(blocks), 1, 1);
  config.blockDim = dim3(kThreads, 1, 1);
  config.dynamicSmemBytes = 0;
  config.stream = stream;
  config.attrs = nullptr;
  config.numAttrs = 0;
  return check_cuda(cudaLaunchKernelEx(&config, allreduce_push_kernel, partial, out, count, rank, world, max_count,
                                       peer_poll_limit(), peers),
                    "peer all-reduce launch");
}

int take_allreduce_status() {
  int status = 0;
  if (cudaMemcpyFromSymbol(&status, g_allreduce_status, sizeof(int)) != cudaSuccess) return -1;
  if (status != 0) {
    const int zero = 0;
    cudaMemcpyToSymbol(g_allreduce_status, &zero, sizeof(int));
  }
  return status;
}

}  // namespace aq
