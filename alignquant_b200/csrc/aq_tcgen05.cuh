// Device helpers for the tcgen05 (tensor-memory) kernels and the host-side tensor-map
// encoder they share.  sm_100a only.
#pragma once

#include <cuda.h>

#include <mutex>

#include "aq_common.cuh"
#include "aq_ptx.cuh"

namespace aq {

#ifdef __CUDACC__
// One box of a 2-D tensor map, global -> shared; x counts elements of the inner
// dimension and x * element size must be a multiple of 16 bytes.
__device__ __forceinline__ void tensor_copy_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(bar)
      : "memory");
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
// Wait for this thread's tensor-memory loads.  The loaded registers are named as operands so
// that the compiler cannot move their uses ahead of the wait.
__device__ __forceinline__ void tc_wait_ld(int (&v)[16]) {
  asm volatile("tcgen05.wait::ld.sync.aligned;"
               : "+r"(v[0]), "+r"(v[1]), "+r"(v[2]), "+r"(v[3]), "+r"(v[4]), "+r"(v[5]), "+r"(v[6]), "+r"(v[7]),
                 "+r"(v[8]), "+r"(v[9]), "+r"(v[10]), "+r"(v[11]), "+r"(v[12]), "+r"(v[13]), "+r"(v[14]), "+r"(v[15])
               :
               : "memory");
}
// A whole warp waits on an mbarrier through one polling lane: thirty-two lanes polling (or
// arriving on) one barrier word are served one after the other by the shared-memory unit,
// which was measured at several hundred cycles per wait.  The shuffle that hands out the
// result is a warp-level synchronisation and orders the other lanes after the poll.
__device__ __forceinline__ bool warp_wait(uint32_t bar, uint32_t parity, int lane, volatile uint32_t* abort_flag,
                                          int* status, int code) {
  int ok = 1;
  if (lane == 0) ok = mbar_wait(bar, parity, abort_flag, status, code) ? 1 : 0;
  return __shfl_sync(0xffffffffu, ok, 0) != 0;
}
// True in exactly one lane of a converged warp.
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "elect.sync _|p, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(pred));
  return pred != 0;
}

// K-major shared-memory operand descriptor with the 64-byte swizzle: a row is 64
// contiguous bytes whose 16-byte chunks are XOR-ed with address bits 7-8, 8-row groups
// are 512 bytes apart (stride byte offset); the leading byte offset is not used by
// swizzled K-major layouts and is encoded as 16 bytes.  Bit 46: sm_100 descriptor format.
__device__ __forceinline__ uint64_t smem_desc_sw64(uint32_t addr) {
  return static_cast<uint64_t>((addr & 0x3ffffu) >> 4) | (static_cast<uint64_t>(16u >> 4) << 16) |
         (static_cast<uint64_t>(512u >> 4) << 32) | (1ull << 46) | (4ull << 61);
}
// kind::i8: D = S32 (2), A = B = signed 8-bit (1), both K-major, M = 128.
__device__ __forceinline__ uint32_t instr_desc_i8(int n) {
  return (2u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(n >> 3) << 17) |
         (static_cast<uint32_t>(128 >> 4) << 24);
}

// Packed FP32 pairs (add.f32x2 / mul.f32x2): the same IEEE round-to-nearest results as the
// scalar instructions at two thirds of the issue slots.
__device__ __forceinline__ uint64_t pack2(uint32_t lo, uint32_t hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(lo), "r"(hi));
  return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}
// There is no packed multiply here on purpose: the assembler contracts a packed multiply
// (however it is written) that feeds a packed add into one fused multiply-add, which
// rounds a * b + c once instead of twice.  The products are therefore formed with the
// scalar instruction, which keeps its own rounding.

#endif  // __CUDACC__

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
inline std::once_flag g_encode_once;
inline EncodeTiledFn g_encode_tiled = nullptr;

// The driver's tensor-map encoder, looked up through the runtime so that the library
// does not link against the driver library.
inline EncodeTiledFn encode_tiled_fn() {
  std::call_once(g_encode_once, [] {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult found = cudaDriverEntryPointSymbolNotFound;
    if (cudaGetDriverEntryPointByVersion("cuTensorMapEncodeTiled", &fn, 12000, cudaEnableDefault, &found) ==
            cudaSuccess &&
        found == cudaDriverEntryPointSuccess) {
      g_encode_tiled = reinterpret_cast<EncodeTiledFn>(fn);
    }
  });
  return g_encode_tiled;
}

// Row-major int8 [m][k] seen as boxes of box_rows rows x 64 bytes that land with the 64-byte
// swizzle; rows past m are filled with zeros.
inline int encode_activation_map(CUtensorMap* map, const int8_t* xq, int64_t m, int64_t k, int box_rows) {
  EncodeTiledFn encode = encode_tiled_fn();
  if (encode == nullptr) return fail(AQ_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(k), static_cast<cuuint64_t>(m)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(k)};
  const cuuint32_t box[2] = {static_cast<cuuint32_t>(kTile), static_cast<cuuint32_t>(box_rows)};
  const cuuint32_t elem_strides[2] = {1, 1};
  const CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<int8_t*>(xq), dims, strides, box,
                            elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B,
                            CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(AQ_ERR_CUDA, "cuTensorMapEncodeTiled failed with code %d", static_cast<int>(r));
  return AQ_OK;
}

}  // namespace aq
