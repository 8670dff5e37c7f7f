// Measurement aid: the rate at which this GPU's tensor cores execute tcgen05.mma kind::i8 when
// nothing else happens -- no operand traffic, no accumulator drain.  It is the denominator of
// the GEMM's tensor-pipe fraction ("measured INT8 peak"), taken on the device and at the clocks
// the GEMM itself runs on.
//
// One CTA per SM.  The operands (a 128 x 64 int8 block and a 256 x 64 int8 block in the K-major
// 64-byte-swizzle layout, all zero) sit in shared memory; one elected thread issues `pairs` x 2
// MMAs of shape M128 N256 K32 back to back into one 256-column tensor-memory accumulator and
// commits once at the end; the CTA waits (bounded) for that commit.  2 * 128 * 256 * 64 integer
// operations per pair.
#include "aq_common.cuh"
#include "aq_ptx.cuh"
#include "aq_tcgen05.cuh"

namespace aq {

__device__ int g_peak_status = 0;

namespace {

constexpr int kPeakThreads = 128;
constexpr int kPeakABytes = 128 * kTile;
constexpr int kPeakBBytes = 256 * kTile;
constexpr int kPeakSmem = kPeakABytes + kPeakBBytes + 1024 + 64;  // operands (1024-byte aligned) + barrier

__global__ void __launch_bounds__(kPeakThreads, 1) int8_peak_kernel(int pairs) {
  extern __shared__ __align__(1024) uint8_t smem[];
  uint64_t* bar = reinterpret_cast<uint64_t*>(smem + kPeakABytes + kPeakBBytes);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar + 1);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < (kPeakABytes + kPeakBBytes) / 16; i += kPeakThreads) {
    reinterpret_cast<uint4*>(smem)[i] = make_uint4(0, 0, 0, 0);
  }
  const uint32_t bar_addr = smem_u32(bar);
  if (threadIdx.x == 0) {
    mbar_init(bar_addr, 1);
    *abort_flag = 0;
    mbar_init_fence();
  }
  fence_proxy_async();  // the zeroed operands become visible to the tensor cores
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(256u)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  if (warp == 0) {
    const uint32_t idesc = instr_desc_i8(256);
    const uint32_t a_addr = smem_u32(smem);
    const uint32_t b_addr = a_addr + kPeakABytes;
    for (int i = 0; i < pairs; ++i) {
      if (elect_one()) {
        tc_mma_i8(tmem_base, smem_desc_sw64(a_addr), smem_desc_sw64(b_addr), idesc, i == 0 ? 0u : 1u);
        tc_mma_i8(tmem_base, smem_desc_sw64(a_addr + 32), smem_desc_sw64(b_addr + 32), idesc, 1u);
      }
      __syncwarp();
    }
    if (elect_one()) tc_commit(bar_addr);
    __syncwarp();
    warp_wait(bar_addr, 0, lane, abort_flag, &g_peak_status, 1);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(256u) : "memory");
  }
}

}  // namespace

// Runs the kernel twice (warm-up, then timed with CUDA events on `stream`), synchronises and
// reports integer tera-operations per second over all SMs.
int measure_int8_peak(int pairs, double* tops, cudaStream_t stream) {
  int rc = check_cuda(cudaFuncSetAttribute(int8_peak_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kPeakSmem),
                      "cudaFuncSetAttribute(int8_peak_kernel)");
  if (rc != AQ_OK) return rc;
  const int sms = num_sms();
  cudaEvent_t begin = nullptr, end = nullptr;
  rc = check_cuda(cudaEventCreate(&begin), "cudaEventCreate");
  if (rc != AQ_OK) return rc;
  rc = check_cuda(cudaEventCreate(&end), "cudaEventCreate");
  if (rc != AQ_OK) {
    cudaEventDestroy(begin);
    return rc;
  }
  float ms = 0.0f;
  int8_peak_kernel<<<sms, kPeakThreads, kPeakSmem, stream>>>(pairs);
  cudaEventRecord(begin, stream);
  int8_peak_kernel<<<sms, kPeakThreads, kPeakSmem, stream>>>(pairs);
  cudaEventRecord(end, stream);
  rc = check_cuda(cudaEventSynchronize(end), "int8 peak kernel");
  if (rc == AQ_OK) rc = check_cuda(cudaEventElapsedTime(&ms, begin, end), "cudaEventElapsedTime");
  cudaEventDestroy(begin);
  cudaEventDestroy(end);
  if (rc != AQ_OK) return rc;
  int status = 0;
  if (cudaMemcpyFromSymbol(&status, g_peak_status, sizeof(int)) == cudaSuccess && status != 0) {
    const int zero = 0;
    cudaMemcpyToSymbol(g_peak_status, &zero, sizeof(int));
    return fail(AQ_ERR_DEVICE, "the int8 peak kernel gave up waiting for its MMAs");
  }
  const double ops = 2.0 * 128.0 * 256.0 * 64.0 * static_cast<double>(pairs) * sms;
  *tops = ops / (static_cast<double>(ms) * 1e-3) / 1e12;
  return AQ_OK;
}

}  // namespace aq
