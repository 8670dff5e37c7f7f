// extern "C" entry points of libalignquant_b200.so: argument validation and dispatch.
// The checks mirror the argument contract of the reference host functions
// (alignquant/kernels/cuda/linear.cu:1520-1533, 1578-1672) in terms of raw pointers.
#include <atomic>
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "aq_common.cuh"

namespace aq {

std::string& last_error_storage() {
  thread_local std::string text;
  return text;
}

int fail(int code, const char* format, ...) {
  char buffer[512];
  va_list args;
  va_start(args, format);
  vsnprintf(buffer, sizeof(buffer), format, args);
  va_end(args);
  last_error_storage() = buffer;
  return code;
}

int check_cuda(cudaError_t status, const char* what) {
  if (status == cudaSuccess) return AQ_OK;
  return fail(AQ_ERR_CUDA, "%s: %s", what, cudaGetErrorString(status));
}

int num_sms() {
  // cached per device; the library may be used from several devices of one process
  static std::mutex mutex;
  static int cached[64] = {0};
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return 148;
  std::lock_guard<std::mutex> lock(mutex);
  if (cached[device] == 0) {
    int value = 0;
    if (cudaDeviceGetAttribute(&value, cudaDevAttrMultiProcessorCount, device) != cudaSuccess ||
        value <= 0) {
      value = 148;
    }
    cached[device] = value;
  }
  return cached[device];
}

bool use_dependent_launch() {
  static const bool enabled = [] {
    const char* value = std::getenv("ALIGNQUANT_B200_PDL");
    return value == nullptr || std::strcmp(value, "0") != 0;
  }();
  return enabled;
}

namespace {
constexpr int64_t kDefaultPeerPollLimit = 1LL << 22;
constexpr int64_t kDefaultQuantFusionTiles = 2400;
std::atomic<int64_t> g_peer_poll_limit{kDefaultPeerPollLimit};
std::atomic<int64_t> g_gemm_rounding{0};
std::atomic<int64_t> g_gemm_tile{0};
std::atomic<int64_t> g_gemm_split{0};
std::atomic<int64_t> g_decode_kernel{0};
std::atomic<int64_t> g_quant_fusion_tiles{kDefaultQuantFusionTiles};
}  // namespace

uint32_t peer_poll_limit() { return static_cast<uint32_t>(g_peer_poll_limit.load(std::memory_order_relaxed)); }
bool gemm_separate_rounding() { return g_gemm_rounding.load(std::memory_order_relaxed) != 0; }
int gemm_tile_option() { return static_cast<int>(g_gemm_tile.load(std::memory_order_relaxed)); }
int gemm_split_option() { return static_cast<int>(g_gemm_split.load(std::memory_order_relaxed)); }
int decode_kernel_option() { return static_cast<int>(g_decode_kernel.load(std::memory_order_relaxed)); }
int64_t quant_fusion_tiles() { return g_quant_fusion_tiles.load(std::memory_order_relaxed); }

namespace {

constexpr int64_t kStreamMaxRows = 128;  // most rows of the streaming cluster kernel (explicit schedules)
constexpr int64_t kAutoGemmRows = 32;    // above this the automatic schedule uses the GEMM (split-K for few rows)
constexpr int64_t kDecodeMaxRows = 16;   // the persistent decode kernel handles up to this many rows
constexpr int64_t kClusterMaxRows = 32;  // the warp-per-tile cluster kernel handles up to this many rows

bool valid_split(int s) { return s == 0 || s == 1 || s == 2 || s == 4 || s == 8 || s == 16; }

// Kernel families (also the values aq_linear_plan reports):
//   0 cluster kernel, eight warps per tile, tiles of a split added in increasing k
//     (explicit split counts, forced non-GEMM schedules up to 128 rows)
//   1 tensor-memory GEMM (K ranges over a cluster where few rows leave SMs idle)
//   2 persistent stream-K kernel (at most 16 rows, layers with very few tile rows)
//   3 cluster kernel, one warp (two for 17..32 rows) per tile: decode sizes, layers too narrow
//     for family 4
//   4 decode kernel of many small CTAs without a K split (reported to callers as kernel 3 with
//     one range): the default decode kernel of layers with enough tile rows and K up to 64 tiles
//     (128 for at most eight rows)
int choose_kernel(int64_t m, int n_j, int n_k, int schedule, int decode_splits) {
  if (schedule == AQ_SCHEDULE_PREFILL_M64) return 1;
  if (schedule == AQ_SCHEDULE_AUTO && (m > kStreamMaxRows || (decode_splits == 0 && m > kAutoGemmRows))) return 1;
  if (decode_splits != 0 || m > kClusterMaxRows) return 0;
  const int64_t wanted = decode_kernel_option();
  if (wanted == AQ_DECODE_KERNEL_STREAMK && m <= kDecodeMaxRows) return 2;
  if (wanted != AQ_DECODE_KERNEL_CLUSTER && direct_decode_supported(m, n_j, n_k)) return 4;
  if (cluster_decode_supported(n_j, n_k)) return 3;
  return m <= kDecodeMaxRows ? 2 : 0;
}

}  // namespace
}  // namespace aq

using namespace aq;

extern "C" {

int aq_version(void) { return 200; }

int aq_set_option(int option, int64_t value) {
  switch (option) {
    case AQ_OPT_PEER_POLL_LIMIT:
      AQ_REQUIRE(value >= 64 && value < (1LL << 31), "AQ_OPT_PEER_POLL_LIMIT must be in [64, 2^31), got %lld",
                 static_cast<long long>(value));
      g_peer_poll_limit.store(value, std::memory_order_relaxed);
      return AQ_OK;
    case AQ_OPT_GEMM_ROUNDING:
      AQ_REQUIRE(value == AQ_GEMM_ROUNDING_FUSED || value == AQ_GEMM_ROUNDING_SEPARATE,
                 "AQ_OPT_GEMM_ROUNDING must be AQ_GEMM_ROUNDING_FUSED or AQ_GEMM_ROUNDING_SEPARATE, got %lld",
                 static_cast<long long>(value));
      g_gemm_rounding.store(value, std::memory_order_relaxed);
      return AQ_OK;
    case AQ_OPT_GEMM_TILE:
      AQ_REQUIRE(value == AQ_GEMM_TILE_AUTO || value == AQ_GEMM_TILE_PAIRED || value == AQ_GEMM_TILE_NARROW ||
                     value == AQ_GEMM_TILE_WIDE,
                 "AQ_OPT_GEMM_TILE must be one of the AQ_GEMM_TILE_* values, got %lld", static_cast<long long>(value));
      g_gemm_tile.store(value, std::memory_order_relaxed);
      return AQ_OK;
    case AQ_OPT_DECODE_KERNEL:
      AQ_REQUIRE(value == AQ_DECODE_KERNEL_AUTO || value == AQ_DECODE_KERNEL_CLUSTER || value == AQ_DECODE_KERNEL_STREAMK,
                 "AQ_OPT_DECODE_KERNEL must be one of the AQ_DECODE_KERNEL_* values, got %lld",
                 static_cast<long long>(value));
      g_decode_kernel.store(value, std::memory_order_relaxed);
      return AQ_OK;
    case AQ_OPT_QUANT_FUSION_TILES:
      AQ_REQUIRE(value >= 0, "AQ_OPT_QUANT_FUSION_TILES must not be negative, got %lld", static_cast<long long>(value));
      g_quant_fusion_tiles.store(value, std::memory_order_relaxed);
      return AQ_OK;
    case AQ_OPT_GEMM_SPLIT:
      AQ_REQUIRE(value >= 0 && value <= 8, "AQ_OPT_GEMM_SPLIT must be 0 (automatic) or 1..8, got %lld",
                 static_cast<long long>(value));
      g_gemm_split.store(value, std::memory_order_relaxed);
      return AQ_OK;
    default:
      return fail(AQ_ERR_INVALID, "unknown option %d", option);
  }
}

int64_t aq_get_option(int option) {
  switch (option) {
    case AQ_OPT_PEER_POLL_LIMIT:
      return g_peer_poll_limit.load(std::memory_order_relaxed);
    case AQ_OPT_GEMM_ROUNDING:
      return g_gemm_rounding.load(std::memory_order_relaxed);
    case AQ_OPT_GEMM_TILE:
      return g_gemm_tile.load(std::memory_order_relaxed);
    case AQ_OPT_GEMM_SPLIT:
      return g_gemm_split.load(std::memory_order_relaxed);
    case AQ_OPT_DECODE_KERNEL:
      return g_decode_kernel.load(std::memory_order_relaxed);
    case AQ_OPT_QUANT_FUSION_TILES:
      return g_quant_fusion_tiles.load(std::memory_order_relaxed);
    default:
      fail(AQ_ERR_INVALID, "unknown option %d", option);
      return AQ_ERR_INVALID;
  }
}

const char* aq_last_error(void) { return last_error_storage().c_str(); }

int aq_quantize_act(const void* x, int x_dtype, int64_t m, int64_t k, const int32_t* v_metadata,
                    int scale_mode, int8_t* q, float* scales, void* stream) {
  AQ_REQUIRE(x != nullptr && q != nullptr && scales != nullptr, "x, q and scales must not be NULL");
  AQ_REQUIRE(m >= 1, "x must have at least one row, got m=%lld", static_cast<long long>(m));
  AQ_REQUIRE(k >= kTile && k % kTile == 0, "K must be a positive multiple of 64, got %lld",
             static_cast<long long>(k));
  AQ_REQUIRE(k <= (1 << 24), "K too large");
  AQ_REQUIRE(scale_mode == AQ_SCALE_TILE || scale_mode == AQ_SCALE_TOKEN,
             "scale_mode must be AQ_SCALE_TILE or AQ_SCALE_TOKEN, got %d", scale_mode);
  AQ_REQUIRE(scale_mode == AQ_SCALE_TILE || v_metadata == nullptr,
             "the structured V transform is only defined for AQ_SCALE_TILE");
  AQ_REQUIRE(aligned(x, 16) && aligned(q, 16), "x and q must be 16-byte aligned for 128-bit access");
  AQ_REQUIRE(aligned(scales, 4) && aligned(v_metadata, 4), "scales and v_metadata must be 4-byte aligned");
  return launch_quantize(x, x_dtype, m, k, v_metadata, scale_mode, q, scales,
                         static_cast<cudaStream_t>(stream));
}

int aq_rmsnorm_quantize(const void* x, int x_dtype, int64_t m, int64_t k, const void* weight, float eps, int8_t* q,
                        float* scales, void* normed, void* stream) {
  AQ_REQUIRE(x != nullptr && weight != nullptr && q != nullptr && scales != nullptr,
             "x, weight, q and scales must not be NULL");
  AQ_REQUIRE(m >= 1, "x must have at least one row, got m=%lld", static_cast<long long>(m));
  AQ_REQUIRE(k >= kTile && k % kTile == 0, "K must be a positive multiple of 64, got %lld", static_cast<long long>(k));
  AQ_REQUIRE(k <= (1 << 24), "K too large");
  AQ_REQUIRE(eps >= 0.0f, "eps must not be negative");
  AQ_REQUIRE(aligned(x, 16) && aligned(weight, 16) && aligned(q, 16) && aligned(normed, 16),
             "x, weight, q and normed must be 16-byte aligned for 128-bit access");
  AQ_REQUIRE(aligned(scales, 4), "scales must be 4-byte aligned");
  return launch_rmsnorm_quantize(x, x_dtype, m, k, weight, eps, q, scales, normed, static_cast<cudaStream_t>(stream));
}

int64_t aq_prepared_bytes(int32_t n_j, int32_t n_k, int64_t t4, int64_t t8) {
  if (n_j <= 0 || n_k <= 0 || t4 < 0 || t8 < 0 || t4 + t8 != static_cast<int64_t>(n_j) * n_k) {
    fail(AQ_ERR_INVALID, "aq_prepared_bytes: need n_j, n_k > 0 and t4 + t8 == n_j * n_k");
    return AQ_ERR_INVALID;
  }
  return records_bytes(t4 + t8) + t4 * kW4TileBytes + t8 * kW8TileBytes;
}

int aq_repack(const uint8_t* state_bits, const uint8_t* w4_payload, const float* w4_scales,
              const int8_t* w8_payload, const float* w8_scales, const int32_t* w4_row_offsets,
              const int32_t* w8_row_offsets, int32_t n_j, int32_t n_k, int64_t t4, int64_t t8,
              void* prepared, int64_t prepared_bytes, void* stream) {
  AQ_REQUIRE(n_j > 0 && n_k > 0, "N and K must contain at least one 64-wide tile");
  AQ_REQUIRE(t4 >= 0 && t8 >= 0 && t4 + t8 == static_cast<int64_t>(n_j) * n_k,
             "selected payload count mismatch: t4 + t8 must equal n_j * n_k");
  AQ_REQUIRE(state_bits != nullptr && w4_row_offsets != nullptr && w8_row_offsets != nullptr,
             "state_bits and row offsets must not be NULL");
  AQ_REQUIRE(t4 == 0 || (w4_payload != nullptr && w4_scales != nullptr), "W4 arena missing");
  AQ_REQUIRE(t8 == 0 || (w8_payload != nullptr && w8_scales != nullptr), "W8 arena missing");
  AQ_REQUIRE(aligned(w4_payload, 8), "w4_payload must be 8-byte aligned");
  AQ_REQUIRE(aligned(w8_payload, 16), "w8_payload must be 16-byte aligned");
  AQ_REQUIRE(prepared != nullptr && aligned(prepared, 256), "prepared image must be 256-byte aligned");
  const int64_t need = aq_prepared_bytes(n_j, n_k, t4, t8);
  if (prepared_bytes < need) {
    return fail(AQ_ERR_WORKSPACE, "prepared image needs %lld bytes, got %lld",
                static_cast<long long>(need), static_cast<long long>(prepared_bytes));
  }
  AQ_REQUIRE(need / kW4TileBytes < (1LL << 31), "layer too large for 31-bit tile offsets");
  return launch_repack(state_bits, w4_payload, w4_scales, w8_payload, w8_scales, w4_row_offsets,
                       w8_row_offsets, n_j, n_k, prepared, static_cast<cudaStream_t>(stream));
}

int64_t aq_linear_workspace_bytes(int64_t m, int32_t n_j, int32_t n_k, int schedule,
                                  int decode_splits) {
  if (m < 1 || n_j <= 0 || n_k <= 0 || schedule < 0 || schedule > 3) {
    fail(AQ_ERR_INVALID, "aq_linear_workspace_bytes: invalid problem");
    return AQ_ERR_INVALID;
  }
  switch (choose_kernel(m, n_j, n_k, schedule, decode_splits)) {
    case 1:
      return tmem_gemm_workspace_bytes(m, n_j, n_k);
    case 2:
      return decode_workspace_bytes(m, n_j, n_k);
    default:
      return 0;
  }
}

}  // extern "C"

struct TensorParallelSum {
  int32_t rank;
  int32_t world;
  void* const* peer_buffers;
  int64_t max_count;
};

struct LookAhead {
  const void* data;
  int64_t bytes;
};

// Activations that are still to be quantized (per-token scales): xq / act_scales of the call are outputs.
struct RawActivation {
  const void* x;
  int dtype;
};

static int linear_impl(const int8_t* xq, const float* act_scales, int scale_mode, int64_t m,
                       const void* prepared, int32_t n_j, int32_t n_k, const int32_t* u_metadata,
                       int schedule, int decode_splits, int out_dtype, void* out, void* workspace,
                       int64_t workspace_bytes, int32_t* acc_dump, const TensorParallelSum* tp,
                       const LookAhead* ahead, void* stream, const RawActivation* raw = nullptr) {
  AQ_REQUIRE(xq != nullptr && act_scales != nullptr && prepared != nullptr && out != nullptr,
             "xq, act_scales, prepared and out must not be NULL");
  AQ_REQUIRE(m >= 1, "x_int8 must have at least one row");
  AQ_REQUIRE(n_j > 0, "N must contain at least one 64-column tile");
  AQ_REQUIRE(n_k > 0, "K must contain at least one 64-column tile");
  AQ_REQUIRE(scale_mode == AQ_SCALE_TILE || scale_mode == AQ_SCALE_TOKEN,
             "scale_mode must be AQ_SCALE_TILE or AQ_SCALE_TOKEN, got %d", scale_mode);
  AQ_REQUIRE(schedule >= 0 && schedule <= 3,
             "schedule must be 0 (auto), 1 (decode), 2 (prefill), or 3 (prefill_m64)");
  AQ_REQUIRE(schedule != AQ_SCHEDULE_DECODE || m == 1,
             "forced decode schedule requires exactly one row");
  AQ_REQUIRE(schedule != AQ_SCHEDULE_PREFILL || m > 1,
             "forced prefill schedule requires more than one row");
  AQ_REQUIRE(schedule != AQ_SCHEDULE_PREFILL_M64 || m > 1,
             "forced M64 prefill schedule requires more than one row");
  AQ_REQUIRE(valid_split(decode_splits), "split override must be 0 (automatic), 1, 2, 4, 8, or 16");
  AQ_REQUIRE(decode_splits == 0 || schedule != AQ_SCHEDULE_PREFILL_M64,
             "split override is not available on the forced M64 prefill schedule");
  AQ_REQUIRE(decode_splits == 0 || decode_splits <= n_k, "decode_splits may not exceed K/64");
  AQ_REQUIRE(out_dtype == AQ_F32 || out_dtype == AQ_BF16 || out_dtype == AQ_F16,
             "out_dtype must be AQ_F32, AQ_BF16 or AQ_F16");
  AQ_REQUIRE(aligned(xq, 16), "x_int8 must be 16-byte aligned for 128-bit access");
  AQ_REQUIRE(aligned(prepared, 256), "prepared image must be 256-byte aligned");
  AQ_REQUIRE(aligned(out, 16), "out must be 16-byte aligned");
  AQ_REQUIRE(aligned(act_scales, 4) && aligned(u_metadata, 4) && aligned(acc_dump, 4),
             "act_scales, u_metadata and acc_dump must be 4-byte aligned");

  const int64_t tiles = static_cast<int64_t>(n_j) * n_k;
  LinearArgs a;
  a.xq = xq;
  a.act_scales = act_scales;
  a.scale_mode = scale_mode;
  a.m = m;
  a.records = static_cast<const TileRecord*>(prepared);
  a.payload = static_cast<const uint8_t*>(prepared) + records_bytes(tiles);
  a.n_j = n_j;
  a.n_k = n_k;
  a.u_metadata = u_metadata;
  a.out_dtype = out_dtype;
  a.out = out;
  a.acc_dump = acc_dump;
  a.workspace = workspace;
  a.workspace_bytes = workspace_bytes;
  if (ahead != nullptr && ahead->data != nullptr && ahead->bytes > 0) {
    AQ_REQUIRE(aligned(ahead->data, 16) && (ahead->bytes & 15) == 0,
               "the look-ahead range must be 16-byte aligned and a multiple of 16 bytes long");
    a.prefetch = ahead->data;
    a.prefetch_bytes = ahead->bytes;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);

  const int kernel = choose_kernel(m, n_j, n_k, schedule, decode_splits);
  if (tp != nullptr) {
    AQ_REQUIRE(kernel == 3 || kernel == 4, "the fused tensor-parallel sum is only available where aq_linear_plan reports kernel 3");
    a.peer_buffers = tp->peer_buffers;
    a.tp_rank = tp->rank;
    a.tp_world = tp->world;
    a.ar_max_count = tp->max_count;
  }
  if (raw != nullptr) {
    // One launch where the small-CTA decode kernel quantizes its own activations, else the
    // quantizer kernel into xq / act_scales first.
    if (kernel == 4 && (raw->dtype == AQ_F16 || raw->dtype == AQ_BF16) && direct_decode_quantizes(m, n_j, n_k)) {
      a.raw_x = raw->x;
      a.raw_dtype = raw->dtype;
    } else {
      const int rc = launch_quantize(raw->x, raw->dtype, m, static_cast<int64_t>(n_k) * 64, nullptr, AQ_SCALE_TOKEN,
                                     const_cast<int8_t*>(xq), const_cast<float*>(act_scales), s);
      if (rc != AQ_OK) return rc;
    }
  }
  if (kernel == 4) return launch_direct_decode(a, s);
  if (kernel == 3) return launch_cluster_decode(a, s);
  if (kernel == 0) {
    AQ_REQUIRE(decode_splits == 0 || m <= kStreamMaxRows,
               "split override requires at most 128 rows");
    const int split = decode_splits != 0 ? decode_splits : stream_auto_split(m, n_j, n_k);
    return launch_stream_linear(a, split, s);
  }
  const int64_t need = kernel == 2 ? decode_workspace_bytes(m, n_j, n_k) : tmem_gemm_workspace_bytes(m, n_j, n_k);
  if (need > 0 && (workspace == nullptr || workspace_bytes < need || !aligned(workspace, 256))) {
    return fail(AQ_ERR_WORKSPACE, "aq_linear needs a 256-byte aligned workspace of %lld bytes",
                static_cast<long long>(need));
  }
  return kernel == 2 ? launch_decode_linear(a, s) : launch_tmem_gemm(a, s);
}


extern "C" {

int aq_linear(const int8_t* xq, const float* act_scales, int scale_mode, int64_t m,
              const void* prepared, int32_t n_j, int32_t n_k, const int32_t* u_metadata,
              int schedule, int decode_splits, int out_dtype, void* out, void* workspace,
              int64_t workspace_bytes, int32_t* acc_dump, void* stream) {
  return linear_impl(xq, act_scales, scale_mode, m, prepared, n_j, n_k, u_metadata, schedule, decode_splits, out_dtype,
                     out, workspace, workspace_bytes, acc_dump, nullptr, nullptr, stream);
}

int aq_linear_ahead(const int8_t* xq, const float* act_scales, int scale_mode, int64_t m,
                    const void* prepared, int32_t n_j, int32_t n_k, const int32_t* u_metadata,
                    int schedule, int decode_splits, int out_dtype, void* out, void* workspace,
                    int64_t workspace_bytes, int32_t* acc_dump, const void* next_prepared,
                    int64_t next_bytes, void* stream) {
  AQ_REQUIRE(next_bytes >= 0, "next_bytes must not be negative");
  const LookAhead ahead = {next_prepared, next_bytes};
  return linear_impl(xq, act_scales, scale_mode, m, prepared, n_j, n_k, u_metadata, schedule, decode_splits, out_dtype,
                     out, workspace, workspace_bytes, acc_dump, nullptr, &ahead, stream);
}

int aq_linear_allreduce(const int8_t* xq, const float* act_scales, int scale_mode, int64_t m,
                        const void* prepared, int32_t n_j, int32_t n_k, const int32_t* u_metadata,
                        int out_dtype, void* out, int32_t rank, int32_t world, void* const* peer_buffers,
                        int64_t max_count, const void* next_prepared, int64_t next_bytes, void* stream) {
  AQ_REQUIRE(next_bytes >= 0, "next_bytes must not be negative");
  AQ_REQUIRE(peer_buffers != nullptr, "peer_buffers must not be NULL");
  AQ_REQUIRE(world >= 2 && world <= allreduce_max_ranks(), "world must be 2..%d, got %d", allreduce_max_ranks(), world);
  AQ_REQUIRE(rank >= 0 && rank < world, "rank must be in [0, world)");
  AQ_REQUIRE(max_count >= 4 && (max_count & 3) == 0, "max_count must be a positive multiple of 4");
  AQ_REQUIRE(m >= 1 && n_j > 0 && m * static_cast<int64_t>(n_j) * 64 <= max_count,
             "the output (m x N values) must fit the exchange buffers (max_count)");
  for (int r = 0; r < world; ++r) {
    AQ_REQUIRE(peer_buffers[r] != nullptr && aligned(peer_buffers[r], 16), "peer_buffers[%d] must be a 16-byte aligned device pointer", r);
  }
  const TensorParallelSum tp = {rank, world, peer_buffers, max_count};
  const LookAhead ahead = {next_prepared, next_bytes};
  return linear_impl(xq, act_scales, scale_mode, m, prepared, n_j, n_k, u_metadata, AQ_SCHEDULE_AUTO, 0, out_dtype, out,
                     nullptr, 0, nullptr, &tp, &ahead, stream);
}

int aq_quant_linear(const void* x, int x_dtype, int64_t m, const void* prepared, int32_t n_j, int32_t n_k,
                    const int32_t* u_metadata, int out_dtype, void* out, int8_t* xq, float* act_scales, void* workspace,
                    int64_t workspace_bytes, int32_t rank, int32_t world, void* const* peer_buffers, int64_t max_count,
                    const void* next_prepared, int64_t next_bytes, void* stream) {
  AQ_REQUIRE(x != nullptr && aligned(x, 16), "x must be a 16-byte aligned device pointer");
  AQ_REQUIRE(x_dtype == AQ_F16 || x_dtype == AQ_BF16 || x_dtype == AQ_F32, "x_dtype must be AQ_F16, AQ_BF16 or AQ_F32, got %d", x_dtype);
  AQ_REQUIRE(next_bytes >= 0, "next_bytes must not be negative");
  const RawActivation raw = {x, x_dtype};
  const LookAhead ahead = {next_prepared, next_bytes};
  if (peer_buffers == nullptr) {
    return linear_impl(xq, act_scales, AQ_SCALE_TOKEN, m, prepared, n_j, n_k, u_metadata, AQ_SCHEDULE_AUTO, 0, out_dtype, out,
                       workspace, workspace_bytes, nullptr, nullptr, &ahead, stream, &raw);
  }
  AQ_REQUIRE(world >= 2 && world <= allreduce_max_ranks(), "world must be 2..%d, got %d", allreduce_max_ranks(), world);
  AQ_REQUIRE(rank >= 0 && rank < world, "rank must be in [0, world)");
  AQ_REQUIRE(max_count >= 4 && (max_count & 3) == 0, "max_count must be a positive multiple of 4");
  AQ_REQUIRE(m >= 1 && n_j > 0 && m * static_cast<int64_t>(n_j) * 64 <= max_count,
             "the output (m x N values) must fit the exchange buffers (max_count)");
  for (int r = 0; r < world; ++r) {
    AQ_REQUIRE(peer_buffers[r] != nullptr && aligned(peer_buffers[r], 16), "peer_buffers[%d] must be a 16-byte aligned device pointer", r);
  }
  const int kernel = (m >= 1 && n_j > 0 && n_k > 0) ? choose_kernel(m, n_j, n_k, AQ_SCHEDULE_AUTO, 0) : -1;
  AQ_REQUIRE(kernel == 3 || kernel == 4, "the fused tensor-parallel sum is only available where aq_linear_plan reports kernel 3");
  const TensorParallelSum tp = {rank, world, peer_buffers, max_count};
  return linear_impl(xq, act_scales, AQ_SCALE_TOKEN, m, prepared, n_j, n_k, u_metadata, AQ_SCHEDULE_AUTO, 0, out_dtype, out,
                     nullptr, 0, nullptr, &tp, &ahead, stream, &raw);
}

int aq_quant_linear_fused(int64_t m, int32_t n_j, int32_t n_k) {
  if (m < 1 || n_j <= 0 || n_k <= 0) return 0;
  return choose_kernel(m, n_j, n_k, AQ_SCHEDULE_AUTO, 0) == 4 && direct_decode_quantizes(m, n_j, n_k) ? 1 : 0;
}

int aq_linear_decode_static(const int8_t* xq, const float* act_scales, int scale_mode, int64_t m,
                            const void* prepared, int32_t n_j, int32_t n_k, const int32_t* u_metadata,
                            int out_dtype, void* out, void* stream) {
  AQ_REQUIRE(xq != nullptr && act_scales != nullptr && prepared != nullptr && out != nullptr,
             "xq, act_scales, prepared and out must not be NULL");
  AQ_REQUIRE(m >= 1 && m <= kDecodeMaxRows, "aq_linear_decode_static handles 1 to %d rows, got %lld",
             static_cast<int>(kDecodeMaxRows), static_cast<long long>(m));
  AQ_REQUIRE(n_j > 0 && n_k > 0, "N and K must contain at least one 64-wide tile");
  AQ_REQUIRE(scale_mode == AQ_SCALE_TILE || scale_mode == AQ_SCALE_TOKEN,
             "scale_mode must be AQ_SCALE_TILE or AQ_SCALE_TOKEN, got %d", scale_mode);
  AQ_REQUIRE(out_dtype == AQ_F32 || out_dtype == AQ_BF16 || out_dtype == AQ_F16,
             "out_dtype must be AQ_F32, AQ_BF16 or AQ_F16");
  AQ_REQUIRE(aligned(xq, 16) && aligned(out, 16), "x_int8 and out must be 16-byte aligned");
  AQ_REQUIRE(aligned(prepared, 256), "prepared image must be 256-byte aligned");
  AQ_REQUIRE(aligned(act_scales, 4) && aligned(u_metadata, 4), "act_scales and u_metadata must be 4-byte aligned");
  const int64_t tiles = static_cast<int64_t>(n_j) * n_k;
  LinearArgs a;
  a.xq = xq;
  a.act_scales = act_scales;
  a.scale_mode = scale_mode;
  a.m = m;
  a.records = static_cast<const TileRecord*>(prepared);
  a.payload = static_cast<const uint8_t*>(prepared) + records_bytes(tiles);
  a.n_j = n_j;
  a.n_k = n_k;
  a.u_metadata = u_metadata;
  a.out_dtype = out_dtype;
  a.out = out;
  a.acc_dump = nullptr;
  a.workspace = nullptr;
  a.workspace_bytes = 0;
  return launch_decode_linear_static(a, static_cast<cudaStream_t>(stream));
}

int aq_linear_plan(int64_t m, int32_t n_j, int32_t n_k, int schedule, int decode_splits, int32_t* kernel,
                   int32_t* splits, int32_t* workers) {
  AQ_REQUIRE(m >= 1 && n_j > 0 && n_k > 0 && schedule >= 0 && schedule <= 3, "aq_linear_plan: invalid problem");
  AQ_REQUIRE(kernel != nullptr && splits != nullptr && workers != nullptr, "aq_linear_plan: NULL output");
  const int k = choose_kernel(m, n_j, n_k, schedule, decode_splits);
  *kernel = k;
  *workers = 1;
  *splits = 1;
  if (k == 0) {
    int s = decode_splits != 0 ? decode_splits : stream_auto_split(m, n_j, n_k);
    if (s > 8) s = 8;
    while (s > n_k) s /= 2;
    *splits = s;  // the launcher may raise it further for very long K; see aq_stream.cu
  } else if (k == 1) {
    *splits = tmem_gemm_split(m, n_j, n_k);
  } else if (k == 2) {
    *splits = decode_ctas(n_j, n_k);
    *workers = 16;
  } else if (k == 3) {
    *splits = cluster_decode_split(m, n_j, n_k);
    *workers = 8;
  } else if (k == 4) {  // same order as kernel 3 with a single K range
    *kernel = 3;
    *splits = 1;
    *workers = direct_decode_workers(m, n_j, n_k);
  }
  return AQ_OK;
}

int64_t aq_allreduce_buffer_bytes(int32_t world, int64_t max_count) {
  if (world < 2 || world > allreduce_max_ranks() || max_count < 4 || (max_count & 3) != 0) {
    fail(AQ_ERR_INVALID, "aq_allreduce_buffer_bytes: world must be 2..%d and max_count a positive multiple of 4",
         allreduce_max_ranks());
    return AQ_ERR_INVALID;
  }
  return allreduce_buffer_bytes(world, max_count);
}

int aq_allreduce_f32(const float* partial, float* out, int64_t count, int32_t rank, int32_t world,
                     void* const* peer_buffers, int64_t max_count, void* stream) {
  AQ_REQUIRE(partial != nullptr && out != nullptr && peer_buffers != nullptr, "partial, out and peer_buffers must not be NULL");
  AQ_REQUIRE(world >= 2 && world <= allreduce_max_ranks(), "world must be 2..%d, got %d", allreduce_max_ranks(), world);
  AQ_REQUIRE(rank >= 0 && rank < world, "rank must be in [0, world)");
  AQ_REQUIRE(max_count >= 4 && (max_count & 3) == 0, "max_count must be a positive multiple of 4");
  AQ_REQUIRE(count >= 4 && (count & 3) == 0 && count <= max_count, "count must be a multiple of 4 in [4, max_count]");
  AQ_REQUIRE(aligned(partial, 16) && aligned(out, 16), "partial and out must be 16-byte aligned");
  for (int r = 0; r < world; ++r) {
    AQ_REQUIRE(peer_buffers[r] != nullptr && aligned(peer_buffers[r], 16), "peer_buffers[%d] must be a 16-byte aligned device pointer", r);
  }
  return launch_allreduce(partial, out, count, rank, world, peer_buffers, max_count, static_cast<cudaStream_t>(stream));
}

int aq_measure_int8_peak(int32_t pairs, double* tops, void* stream) {
  AQ_REQUIRE(tops != nullptr, "tops must not be NULL");
  AQ_REQUIRE(pairs >= 16 && pairs <= (1 << 20), "pairs must be in [16, 2^20], got %d", pairs);
  return measure_int8_peak(pairs, tops, static_cast<cudaStream_t>(stream));
}

int aq_device_status(void* stream) {
  const int rc = check_cuda(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)), "cudaStreamSynchronize");
  if (rc != AQ_OK) return rc;
  const int stream_status = take_stream_status();
  const int gemm_status = take_gemm_status();
  const int decode_status = take_decode_status();
  const int direct_status = take_direct_decode_status();
  int cluster_decode_status = take_cluster_decode_status();
  if (cluster_decode_status == 0) cluster_decode_status = direct_status;  // both report the fused rank sum's waits
  const int allreduce_status = take_allreduce_status();
  if (allreduce_status > 0) {
    return fail(AQ_ERR_DEVICE, "the peer all-reduce gave up waiting for rank %d; its output is invalid", allreduce_status - 1);
  }
  if (stream_status < 0 || gemm_status < 0 || decode_status < 0 || cluster_decode_status < 0 || allreduce_status < 0) {
    return fail(AQ_ERR_CUDA, "could not read the device status words");
  }
  if (stream_status != 0 || gemm_status != 0 || decode_status != 0 || cluster_decode_status != 0) {
    return fail(AQ_ERR_DEVICE,
                "a kernel wait timed out on the device (wait ids: cluster kernels %d/%d, GEMM %d, stream-K kernel %d); "
                "outputs of that launch are invalid and any workspace must be zeroed again",
                stream_status, cluster_decode_status, gemm_status, decode_status);
  }
  return AQ_OK;
}

}  // extern "C"
