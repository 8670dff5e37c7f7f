// Shared declarations of the alignquant_b200 CUDA library (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <string>

#include "../../include/alignquant_b200.h"

namespace aq {

constexpr int kTile = 64;
constexpr int kW4TileBytes = 2048;
constexpr int kW8TileBytes = 4096;
constexpr uint32_t kW4Flag = 0x80000000u;

// One 8-byte record per weight tile of the prepared image.
struct __align__(8) TileRecord {
  uint32_t offset_flag;  // payload offset / 2048, bit 31 set for W4
  float scale;           // W8: tile scale; W4: tile scale / 16 (kernels feed 16*w to the MMA)
};

inline int64_t records_bytes(int64_t tiles) {
  const int64_t raw = tiles * static_cast<int64_t>(sizeof(TileRecord));
  return (raw + kW4TileBytes - 1) / kW4TileBytes * kW4TileBytes;
}

// ---- error reporting -------------------------------------------------------
std::string& last_error_storage();
int fail(int code, const char* format, ...);
int check_cuda(cudaError_t status, const char* what);

#define AQ_REQUIRE(cond, ...)                         \
  do {                                                \
    if (!(cond)) return ::aq::fail(AQ_ERR_INVALID, __VA_ARGS__); \
  } while (0)

inline bool aligned(const void* p, size_t a) {
  return (reinterpret_cast<uintptr_t>(p) % a) == 0;
}

int num_sms();

// ---- kernel launchers (one per translation unit) ----------------------------
int launch_quantize(const void* x, int x_dtype, int64_t m, int64_t k, const int32_t* v_metadata,
                    int scale_mode, int8_t* q, float* scales, cudaStream_t stream);

int launch_rmsnorm_quantize(const void* x, int x_dtype, int64_t m, int64_t k, const void* weight, float eps, int8_t* q,
                            float* scales, void* normed, cudaStream_t stream);

int launch_repack(const uint8_t* state_bits, const uint8_t* w4_payload, const float* w4_scales,
                  const int8_t* w8_payload, const float* w8_scales, const int32_t* w4_row_offsets,
                  const int32_t* w8_row_offsets, int n_j, int n_k, void* prepared,
                  cudaStream_t stream);

struct LinearArgs {
  const int8_t* xq;
  const float* act_scales;
  int scale_mode;
  int64_t m;
  const TileRecord* records;
  const uint8_t* payload;
  int n_j;
  int n_k;
  const int32_t* u_metadata;
  int out_dtype;
  void* out;
  int32_t* acc_dump;
  void* workspace;
  int64_t workspace_bytes;
  // Row-parallel layer under tensor parallelism: sum the ranks' outputs inside the kernel
  // through the peer exchange buffers of aq_allreduce_f32 (tp_world <= 1: off).
  void* const* peer_buffers = nullptr;
  int tp_rank = 0;
  int tp_world = 1;
  int64_t ar_max_count = 0;
  // Look-ahead: bytes of this GPU's memory (the prepared image of the projection that runs
  // next) that the decode kernels ask the L2 cache to fetch while they run; nullptr: none.
  const void* prefetch = nullptr;
  int64_t prefetch_bytes = 0;
  // Unquantized activations (fp16 / bf16 rows) for a kernel that quantizes them itself; xq and
  // act_scales are then outputs.  nullptr: the activations are in xq / act_scales already.
  const void* raw_x = nullptr;
  int raw_dtype = 0;
};

// Layout of a peer exchange buffer (shared by aq_allreduce.cu and the fused decode epilogue):
// [uint32 call counter, uint32 CTA counter | pad to kArHeaderBytes |
//  recv[2][world][max_count] x {float value, uint32 call number}]
constexpr int kArHeaderBytes = 1024;
constexpr int kArMaxRanks = 8;
struct ArPeers {
  uint8_t* buffer[kArMaxRanks];
};

// Streaming kernel for small m (mma.sync, split-K reduced through cluster shared memory).
int launch_stream_linear(const LinearArgs& a, int split_k, cudaStream_t stream);
int stream_auto_split(int64_t m, int n_j, int n_k);

// Warp-per-tile cluster kernel for m <= 16 (the default decode kernel).
int launch_cluster_decode(const LinearArgs& a, cudaStream_t stream);
int cluster_decode_split(int64_t m, int n_j, int n_k);
bool cluster_decode_supported(int n_j, int n_k);
int take_cluster_decode_status();

// Decode kernel of many small CTAs without a K split for m <= 32: layers with enough column
// groups to fill the machine and K short enough for a CTA's block to fit shared memory.
int launch_direct_decode(const LinearArgs& a, cudaStream_t stream);
bool direct_decode_supported(int64_t m, int n_j, int n_k);
int direct_decode_workers(int64_t m, int n_j, int n_k);
bool direct_decode_quantizes(int64_t m, int n_j, int n_k);
int take_direct_decode_status();

// Persistent stream-K kernel for m <= 16 (needs a zeroed, self-cleaning workspace).
int launch_decode_linear(const LinearArgs& a, cudaStream_t stream);
int64_t decode_workspace_bytes(int64_t m, int n_j, int n_k);
int decode_ctas(int n_j, int n_k);
int take_decode_status();
// Same kernel on the library's built-in scratch array (no caller workspace).
int launch_decode_linear_static(const LinearArgs& a, cudaStream_t stream);
int64_t decode_static_scratch_bytes();

// Tensor-memory GEMM (tcgen05) for large m.
int launch_tmem_gemm(const LinearArgs& a, cudaStream_t stream);
int64_t tmem_gemm_workspace_bytes(int64_t m, int n_j, int n_k);
int tmem_gemm_split(int64_t m, int n_j, int n_k);  // K ranges (cluster size) the GEMM will use

// Rate of back-to-back tcgen05.mma kind::i8 on all SMs (measurement aid; synchronises).
int measure_int8_peak(int pairs, double* tops, cudaStream_t stream);

// Sum of per-rank partial outputs through peer memory (one node, one process per GPU).
int launch_allreduce(const float* partial, float* out, int64_t count, int rank, int world, void* const* peer_buffers,
                     int64_t max_count, cudaStream_t stream);
int64_t allreduce_buffer_bytes(int world, int64_t max_count);
int allreduce_max_ranks();
int take_allreduce_status();
// Read and clear the device-side time-out word of each kernel family (0 = none,
// -1 = the word could not be read).
int take_stream_status();
int take_gemm_status();
// Library options (aq_set_option): polls of a peer's data before a tensor-parallel sum gives
// up, and whether the GEMM rounds multiply and add separately.
uint32_t peer_poll_limit();
bool gemm_separate_rounding();
int gemm_tile_option();   // AQ_GEMM_TILE_*
int gemm_split_option();  // 0 = automatic, 1..8 forced
int decode_kernel_option();  // AQ_DECODE_KERNEL_*
int64_t quant_fusion_tiles();  // AQ_OPT_QUANT_FUSION_TILES
// Whether kernels are launched with programmatic stream serialization (dependent
// launch); on by default, ALIGNQUANT_B200_PDL=0 turns it off.
bool use_dependent_launch();

// ---- device helpers -----------------------------------------------------------
#ifdef __CUDACC__

__device__ __forceinline__ float to_float(__half v) { return __half2float(v); }
__device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ float to_float(float v) { return v; }

template <typename T>
__device__ __forceinline__ void store_out(T* out, int64_t index, float value);
template <>
__device__ __forceinline__ void store_out<float>(float* out, int64_t index, float value) {
  out[index] = value;
}
template <>
__device__ __forceinline__ void store_out<__half>(__half* out, int64_t index, float value) {
  out[index] = __float2half_rn(value);
}
template <>
__device__ __forceinline__ void store_out<__nv_bfloat16>(__nv_bfloat16* out, int64_t index,
                                                         float value) {
  out[index] = __float2bfloat16_rn(value);
}

// 64-point unnormalised Walsh-Hadamard transform of one row held by a warp:
// lane l owns elements l (low) and l + 32 (high).
__device__ __forceinline__ void fwht64_warp(double& low, double& high, int lane) {
#pragma unroll
  for (int stride = 1; stride < 32; stride <<= 1) {
    const double low_peer = __shfl_xor_sync(0xffffffffu, low, stride);
    const double high_peer = __shfl_xor_sync(0xffffffffu, high, stride);
    low = (lane & stride) ? low_peer - low : low + low_peer;
    high = (lane & stride) ? high_peer - high : high + high_peer;
  }
  const double a = low, b = high;
  low = a + b;
  high = a - b;
}

// Inverse output transform of one 64-column row held by a warp (lane l owns columns
// l and l + 32): out[r] = left[r] * ((acc * right) H)[perm[r]] / 8, evaluated in FP64
// (alignquant/kernels/cuda/linear.cu:404-430, 1003-1036).  `meta` points at the
// [4][64] int32 rows (mode, permutation, left sign, right sign) of the tile.
__device__ __forceinline__ void inverse_u_row(float& lo, float& hi, const int32_t* meta, int lane) {
  double dl = static_cast<double>(lo) * static_cast<double>(meta[3 * kTile + lane]);
  double dh = static_cast<double>(hi) * static_cast<double>(meta[3 * kTile + lane + 32]);
  fwht64_warp(dl, dh, lane);
  const int t_lo = meta[kTile + lane];
  const int t_hi = meta[kTile + lane + 32];
  const double lo_from_l = __shfl_sync(0xffffffffu, dl, t_lo & 31);
  const double lo_from_h = __shfl_sync(0xffffffffu, dh, t_lo & 31);
  const double hi_from_l = __shfl_sync(0xffffffffu, dl, t_hi & 31);
  const double hi_from_h = __shfl_sync(0xffffffffu, dh, t_hi & 31);
  lo = static_cast<float>((t_lo < 32 ? lo_from_l : lo_from_h) *
                          static_cast<double>(meta[2 * kTile + lane]) * 0.125);
  hi = static_cast<float>((t_hi < 32 ? hi_from_l : hi_from_h) *
                          static_cast<double>(meta[2 * kTile + lane + 32]) * 0.125);
}

#endif  // __CUDACC__

}  // namespace aq
