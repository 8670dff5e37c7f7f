// Sum of the partial outputs of a row-parallel projection over the ranks of one node,
// through peer memory (NVLink / NVSwitch), for the small messages of decode
// (reference: dist.all_reduce after a row-parallel linear, alignquant/quantization/model.py:352-356).
//
// Every rank owns one "exchange buffer" that all peers have mapped:
//   [ counters[kBlocks] | flags[kMaxRanks][kBlocks] | pad to 1024 B | recv[2][world][max_count] floats ]
// One launch per rank and all-reduce, kBlocks CTAs, each CTA owning a contiguous slice:
//   1. epoch = counters[b] + 1 (the number of this all-reduce; lives on the device, so a
//      captured launch can be replayed), parity = epoch & 1;
//   2. push: the CTA stores its slice of the partial into recv[parity][rank] of every peer
//      (plain 16-byte stores that travel over NVLink), then one thread makes them visible
//      (system-scope fence) and writes `epoch` into flags[rank][b] of every peer;
//   3. wait: one thread per peer polls the local flags[peer][b] until it reaches `epoch`.
//      The poll is bounded: on a time-out the CTA records it in a status word and goes on,
//      so a missing peer turns into an error code instead of a hang;
//   4. sum in rank order 0..world-1 (own slice from the partial, the others from the local
//      recv[parity]), which gives every rank the same bits, and store the result.
// Two recv halves are enough: a rank can only reach all-reduce e+2 after every peer has
// signalled e+1, which a peer does after it has finished reading e.
// Only plain peer loads/stores are used: no multicast objects, no multimem.
#include "aq_common.cuh"

namespace aq {

__device__ int g_allreduce_status = 0;

namespace {

constexpr int kBlocks = 16;
constexpr int kMaxRanks = 8;
constexpr int kThreads = 256;
constexpr int kHeaderBytes = 1024;
constexpr uint32_t kPollLimit = 1u << 22;
static_assert((kBlocks + kMaxRanks * kBlocks) * 4 <= kHeaderBytes, "header too small");

struct Peers {
  uint8_t* buffer[kMaxRanks];
};

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__global__ void __launch_bounds__(kThreads) allreduce_push_kernel(const float* __restrict__ partial,
                                                                  float* __restrict__ out, int64_t count,
                                                                  int rank, int world, int64_t max_count,
                                                                  const Peers peers) {
  __shared__ uint32_t epoch_shared;
  const int b = blockIdx.x;
  uint8_t* mine = peers.buffer[rank];
  uint32_t* counters = reinterpret_cast<uint32_t*>(mine);
  uint32_t* flags = counters + kBlocks;  // [kMaxRanks][kBlocks], written by the peers
  if (threadIdx.x == 0) epoch_shared = counters[b] + 1;
  __syncthreads();
  const uint32_t epoch = epoch_shared;
  const int64_t half = static_cast<int64_t>(epoch & 1u) * world * max_count;

  // slice of this CTA, in 16-byte units (count is a multiple of 4)
  const int64_t vec_total = count >> 2;
  const int64_t per_block = (vec_total + kBlocks - 1) / kBlocks;
  const int64_t v_begin = b * per_block;
  const int64_t v_end = v_begin + per_block < vec_total ? v_begin + per_block : vec_total;

  const float4* src = reinterpret_cast<const float4*>(partial);
  for (int step = 1; step < world; ++step) {
    const int peer = (rank + step) % world;  // every rank starts with a different peer
    float4* dst = reinterpret_cast<float4*>(peers.buffer[peer] + kHeaderBytes) + ((half + rank * max_count) >> 2);
    for (int64_t i = v_begin + threadIdx.x; i < v_end; i += kThreads) dst[i] = src[i];
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    for (int step = 1; step < world; ++step) {
      const int peer = (rank + step) % world;
      uint32_t* peer_flags = reinterpret_cast<uint32_t*>(peers.buffer[peer]) + kBlocks;
      st_release_sys(peer_flags + rank * kBlocks + b, epoch);
    }
  }
  if (threadIdx.x < world && threadIdx.x != rank) {
    const uint32_t* flag = flags + threadIdx.x * kBlocks + b;
    uint32_t polls = 0;
    while (static_cast<int32_t>(ld_acquire_sys(flag) - epoch) < 0) {
      if (++polls >= kPollLimit) {
        atomicCAS(&g_allreduce_status, 0, 1 + static_cast<int>(threadIdx.x));
        break;
      }
      if (polls > 64) __nanosleep(100);
    }
  }
  __syncthreads();

  const float4* recv = reinterpret_cast<const float4*>(mine + kHeaderBytes) + (half >> 2);
  float4* dst = reinterpret_cast<float4*>(out);
  for (int64_t i = v_begin + threadIdx.x; i < v_end; i += kThreads) {
    float4 acc = rank == 0 ? src[i] : recv[i];
    for (int r = 1; r < world; ++r) {
      const float4 v = r == rank ? src[i] : recv[(static_cast<int64_t>(r) * max_count >> 2) + i];
      acc.x = __fadd_rn(acc.x, v.x);
      acc.y = __fadd_rn(acc.y, v.y);
      acc.z = __fadd_rn(acc.z, v.z);
      acc.w = __fadd_rn(acc.w, v.w);
    }
    dst[i] = acc;
  }
  if (threadIdx.x == 0) counters[b] = epoch;
}

}  // namespace

int64_t allreduce_buffer_bytes(int world, int64_t max_count) {
  return kHeaderBytes + 2 * static_cast<int64_t>(world) * max_count * static_cast<int64_t>(sizeof(float));
}

int allreduce_max_ranks() { return kMaxRanks; }

int launch_allreduce(const float* partial, float* out, int64_t count, int rank, int world, void* const* peer_buffers,
                     int64_t max_count, cudaStream_t stream) {
  Peers peers;
  for (int r = 0; r < kMaxRanks; ++r) peers.buffer[r] = r < world ? static_cast<uint8_t*>(peer_buffers[r]) : nullptr;
  allreduce_push_kernel<<<kBlocks, kThreads, 0, stream>>>(partial, out, count, rank, world, max_count, peers);
  return check_cuda(cudaGetLastError(), "peer all-reduce launch");
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
