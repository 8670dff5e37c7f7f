/*
 * alignquant_b200 -- C ABI of the B200 (sm_100a) mixed W4/W8-A8 linear-layer path.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream (passed
 * as void*, i.e. a cudaStream_t; NULL is the legacy default stream).  The caller
 * owns every buffer: inputs, outputs, the prepared weight image and the optional
 * workspace.  Calls are asynchronous on the given stream, never synchronise and
 * never allocate.  They return AQ_OK (0) or a negative AQ_ERR_* code; the text of
 * the last error of the calling thread is returned by aq_last_error().  No C++
 * exception crosses this boundary.
 *
 * The functions replace the two host entry points of the reference extension
 * (alignquant/kernels/cuda/linear.cu:1516 and :1564, exported to Python by
 * alignquant/kernels/cuda/bindings.cu:27-52) and the kernels behind them.
 */
#ifndef ALIGNQUANT_B200_H_
#define ALIGNQUANT_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define AQ_API __attribute__((visibility("default")))
#else
#define AQ_API
#endif

#define AQ_OK 0
#define AQ_ERR_INVALID (-1)   /* an argument violates the documented contract        */
#define AQ_ERR_CUDA (-2)      /* a CUDA runtime call or kernel launch failed          */
#define AQ_ERR_WORKSPACE (-3) /* workspace or image buffer smaller than required      */
#define AQ_ERR_DEVICE (-4)    /* a kernel reported a device-side time-out             */

/* element types of activations and outputs */
#define AQ_F16 0
#define AQ_BF16 1
#define AQ_F32 2

/* activation scale granularity */
#define AQ_SCALE_TILE 0  /* one scale per 16-row x 64-column activation tile (reference
                            contract, alignquant/kernels/cuda/linear.cu:546-584)      */
#define AQ_SCALE_TOKEN 1 /* one scale per activation row (benchmark-config contract) */

/* schedule codes, same numbering as alignquant/kernels/cuda/extension.py:290-295 */
#define AQ_SCHEDULE_AUTO 0
#define AQ_SCHEDULE_DECODE 1      /* streaming kernel, requires m == 1                */
#define AQ_SCHEDULE_PREFILL 2     /* streaming kernel, requires m > 1                 */
#define AQ_SCHEDULE_PREFILL_M64 3 /* tensor-memory GEMM kernel, requires m > 1        */

/* Library version: major * 10000 + minor * 100 + patch. */
AQ_API int aq_version(void);

/*
 * Process-wide options.  The reference has no counterpart (its kernels have no device-side
 * waits and one fixed FP32 operation order).
 *   AQ_OPT_PEER_POLL_LIMIT  how often a tensor-parallel sum (aq_allreduce_f32, aq_linear_allreduce)
 *                           polls for a peer's data before it gives up and reports AQ_ERR_DEVICE
 *                           through aq_device_status; 64 .. 2^31-1, default 2^22 (seconds).  Takes
 *                           effect for launches issued after the call.
 *   AQ_OPT_GEMM_ROUNDING    how the tensor-memory GEMM (aq_linear_plan kernel 1) adds a K64 tile:
 *                           AQ_GEMM_ROUNDING_FUSED (default): acc = fma(float(int32), a*w, acc),
 *                           one rounding per tile; AQ_GEMM_ROUNDING_SEPARATE: multiply and add
 *                           rounded separately, the operation order of the reference kernels
 *                           (alignquant/kernels/cuda/linear.cu:956-963), about 20 % slower.  The
 *                           per-tile int32 sums are exact either way.
 *   AQ_OPT_GEMM_TILE        CTA tile of the GEMM, for tests and measurements: AQ_GEMM_TILE_AUTO
 *                           (default), AQ_GEMM_TILE_PAIRED (128 columns, two 256-thread CTAs per
 *                           SM), AQ_GEMM_TILE_NARROW (128 columns, one 512-thread CTA per SM),
 *                           AQ_GEMM_TILE_WIDE (256 columns, one CTA per SM).  Results are
 *                           bit-identical across the three.
 *   AQ_OPT_GEMM_SPLIT       number of K ranges of the GEMM (1..8), 0 = automatic (default); changes
 *                           the FP32 summation order as aq_linear_plan reports.
 *   AQ_OPT_DECODE_KERNEL    AQ_DECODE_KERNEL_AUTO (default); AQ_DECODE_KERNEL_CLUSTER: never use
 *                           the decode kernel of many small CTAs; AQ_DECODE_KERNEL_STREAMK: the
 *                           persistent stream-K kernel for every problem of at most 16 rows (the
 *                           kernel behind aq_linear_decode_static; the automatic choice no longer
 *                           takes it where another kernel applies).  For tests and measurements;
 *                           changes the FP32 summation order as aq_linear_plan reports.
 *   AQ_OPT_QUANT_FUSION_TILES  aq_quant_linear runs as one launch only for layers of at most this
 *                           many 64 x 64 tiles (0: never; default 2400).  While a separate quantizer
 *                           runs, the projection that follows is already fetching its weights, so
 *                           for a layer of several megabytes the two launches are the faster form;
 *                           for a megabyte or two (shards under tensor parallelism) one launch is.
 * aq_set_option returns AQ_OK or AQ_ERR_INVALID; aq_get_option the value or AQ_ERR_INVALID.
 */
#define AQ_OPT_PEER_POLL_LIMIT 1
#define AQ_OPT_GEMM_ROUNDING 2
#define AQ_OPT_GEMM_TILE 3
#define AQ_OPT_GEMM_SPLIT 4
#define AQ_OPT_DECODE_KERNEL 5
#define AQ_OPT_QUANT_FUSION_TILES 6
#define AQ_DECODE_KERNEL_AUTO 0
#define AQ_DECODE_KERNEL_CLUSTER 1
#define AQ_DECODE_KERNEL_STREAMK 2
#define AQ_GEMM_ROUNDING_FUSED 0
#define AQ_GEMM_ROUNDING_SEPARATE 1
#define AQ_GEMM_TILE_AUTO 0
#define AQ_GEMM_TILE_PAIRED 1
#define AQ_GEMM_TILE_NARROW 2
#define AQ_GEMM_TILE_WIDE 4
AQ_API int aq_set_option(int option, int64_t value);
AQ_API int64_t aq_get_option(int option);

/* Text of the last error raised on the calling thread ("" if none). */
AQ_API const char* aq_last_error(void);

/*
 * Activation quantizer: x[m][k] (AQ_F16 / AQ_BF16 / AQ_F32, row-major) -> q[m][k]
 * int8 plus float32 scales.  Replaces alignquant_activation_quantize_cuda,
 * alignquant/kernels/cuda/linear.cu:1516-1562 (kernel :502-603).
 *
 *   v_metadata  int32 [k/64][4][64]: rows (mode, permutation, left sign, right sign)
 *               of the structured 64-point transform applied to every 64-column
 *               block before quantisation; mode 0 = identity.  May be NULL
 *               (all identity).  Only used with AQ_SCALE_TILE.
 *   scale_mode  AQ_SCALE_TILE : scales[ceil(m/16)][k/64]; scale =
 *                               max(max(+v)/127, max(-v)/128, 1e-12) over the tile,
 *                               q = rint(v/scale) in FP64, clamp [-128,127].
 *               AQ_SCALE_TOKEN: scales[m]; scale = max(absmax(row)/127, 1e-12),
 *                               q = rint(x/scale) in IEEE float32, clamp [-127,127].
 *   Requirements: m >= 1, k % 64 == 0, x/q 16-byte aligned.
 */
AQ_API int aq_quantize_act(const void* x, int x_dtype, int64_t m, int64_t k,
                    const int32_t* v_metadata, int scale_mode,
                    int8_t* q, float* scales, void* stream);

/*
 * RMSNorm followed by the per-token activation quantizer (AQ_SCALE_TOKEN) in one kernel, for the
 * two places of a decoder layer where a norm feeds quantized projections (qkv, gate/up).  It
 * replaces the normalisation module plus the quantizer call the reference makes per group
 * (alignquant/quantization/model.py:329-331) and saves a launch and a pass over the activations.
 *   x, weight   x_dtype (AQ_F16 / AQ_BF16 / AQ_F32): x[m][k] row-major, weight[k]
 *   arithmetic  r = float(1 / sqrt(sum(x^2)/k + eps)) with sum, division and root in FP64;
 *               n = round(x * r) to x_dtype; y = round(weight * n) to x_dtype (the Llama / Qwen3
 *               RMSNorm module); scales[row] = max(absmax(y)/127, 1e-12); q = rint(y/scale) in
 *               IEEE float32, clamp [-127, 127]
 *   normed      NULL, or x_dtype [m][k]: also receives y (for consumers other than the projections)
 *   Requirements: m >= 1, k % 64 == 0, pointers 16-byte aligned.
 */
AQ_API int aq_rmsnorm_quantize(const void* x, int x_dtype, int64_t m, int64_t k, const void* weight,
                        float eps, int8_t* q, float* scales, void* normed, void* stream);

/*
 * Size in bytes of the prepared weight image of a layer with n_j x n_k tiles of
 * which t4 are W4 and t8 are W8 (t4 + t8 == n_j * n_k).
 */
AQ_API int64_t aq_prepared_bytes(int32_t n_j, int32_t n_k, int64_t t4, int64_t t8);

/*
 * One-time re-layout of the seven artifact tensors of a layer (device pointers,
 * formats of alignquant/quantization/artifact.py:23-31,131-199: Layout-B tiles,
 * low-nibble-first W4, LSB-first state bitmap with 1 = W4, per-precision arenas
 * with row-offset prefixes) into the image the kernels stream.  Replaces the
 * per-call work of expand_mixed_payload_to_w8_kernel and the per-thread bitmap
 * scans (alignquant/kernels/cuda/linear.cu:166-220, 1242-1256).
 *
 * Image: n_j*n_k 8-byte tile records {uint32 offset/2048 | W4 flag in bit 31,
 * float32 scale (W4: scale/16)}, padded to 2048 bytes, followed by the tiles in
 * (j, k) order.  W8 tile = 4096 B: 64 rows (output column n) of 64 bytes, the 16-byte
 * chunk c = k/16 of row n stored at slot c ^ ((n/2) % 4).  W4 tile = 2048 B: 64 rows of
 * 32 bytes, byte 16h+i of row n = (w[n][32h+i] & 15) | (w[n][32h+16+i] << 4).
 * `prepared` must be 256-byte aligned and at least aq_prepared_bytes() long.
 */
AQ_API int aq_repack(const uint8_t* state_bits, const uint8_t* w4_payload, const float* w4_scales,
              const int8_t* w8_payload, const float* w8_scales,
              const int32_t* w4_row_offsets, const int32_t* w8_row_offsets,
              int32_t n_j, int32_t n_k, int64_t t4, int64_t t8,
              void* prepared, int64_t prepared_bytes, void* stream);

/*
 * Bytes of workspace aq_linear needs for this problem (0 when none is needed).  The
 * workspace holds per-row arrival counters (its first 64 KiB) followed by split-K
 * partial tiles.  Its owner must zero it once before the first call; every call
 * returns the counters to zero, so one buffer can be reused by later calls on the same
 * stream, for any layer.  Calls that may run concurrently (other
 * streams) need separate workspaces.  After an AQ_ERR_DEVICE report zero it again.
 * Replaces the per-call torch::empty of partial planes in the reference
 * (alignquant/kernels/cuda/linear.cu:1692-1695).
 */
AQ_API int64_t aq_linear_workspace_bytes(int64_t m, int32_t n_j, int32_t n_k, int schedule,
                                  int decode_splits);

/*
 * out[m][64*n_j] = sum over K64 tiles of float(int32 tile dot product) *
 * (activation scale * tile scale), accumulated in FP32 in increasing k, followed
 * by the structured inverse output transform.  Replaces alignquant_linear_cuda,
 * alignquant/kernels/cuda/linear.cu:1564-1778, and the kernels it dispatches
 * (:617-698, :700-793, :798-1047, :1053-1210, :1216-1354).
 *
 *   xq            int8 [m][64*n_k] row-major, 16-byte aligned
 *   act_scales    float32, AQ_SCALE_TILE: [ceil(m/16)][n_k]; AQ_SCALE_TOKEN: [m]
 *   prepared      image written by aq_repack
 *   u_metadata    int32 [n_j][4][64] inverse-output-transform rows, or NULL (identity)
 *   schedule      AQ_SCHEDULE_*; decode_splits 0 (automatic) or 1, 2, 4, 8, 16
 *                 (only with AQ_SCHEDULE_AUTO/DECODE/PREFILL and m <= 128;
 *                 values above 8 run as 8)
 *   out_dtype     AQ_F32, AQ_BF16 or AQ_F16; out is [m][64*n_j], 16-byte aligned
 *   workspace     at least aq_linear_workspace_bytes() bytes, 256-byte aligned and
 *                 zeroed by its owner (see above), or NULL when that is 0
 *   acc_dump      NULL, or int32 [m][n_j][n_k][64]: receives every per-tile integer
 *                 dot product (debug/verification aid; slows the call down)
 */
AQ_API int aq_linear(const int8_t* xq, const float* act_scales, int scale_mode, int64_t m,
              const void* prepared, int32_t n_j, int32_t n_k, const int32_t* u_metadata,
              int schedule, int decode_splits, int out_dtype, void* out,
              void* workspace, int64_t workspace_bytes, int32_t* acc_dump, void* stream);

/*
 * aq_linear with a look-ahead: while this projection runs, the decode kernels whose own traffic
 * leaves HBM idle (the many-small-CTA kernel of layers with few tile rows and the stream-K kernel;
 * the others ignore the hint) ask the L2 cache to fetch next_bytes bytes at next_prepared --
 * normally the prepared image of the projection that the caller runs next (aq_prepared_bytes
 * long).  A decode-size projection is a few microseconds of HBM traffic, less than a kernel's
 * chain of latencies; with the look-ahead HBM keeps streaming through them and the next kernel
 * finds its weights on chip.  The range must lie in
 * this GPU's own memory, be 16-byte aligned and a multiple of 16 bytes long; it is only read.
 * next_prepared == NULL or next_bytes == 0: exactly aq_linear.  The reference has no
 * counterpart (its decode kernels read weights straight from HBM,
 * alignquant/kernels/cuda/linear.cu:1216-1313).
 */
AQ_API int aq_linear_ahead(const int8_t* xq, const float* act_scales, int scale_mode, int64_t m,
                    const void* prepared, int32_t n_j, int32_t n_k, const int32_t* u_metadata,
                    int schedule, int decode_splits, int out_dtype, void* out,
                    void* workspace, int64_t workspace_bytes, int32_t* acc_dump,
                    const void* next_prepared, int64_t next_bytes, void* stream);

/*
 * aq_linear for callers that have no way to supply a workspace.  (No counterpart in the
 * reference, whose host function allocates its temporaries itself.)
 *
 * Some hosts of this library can pass in inputs and outputs but nothing else: operator
 * plug-in interfaces whose call signature is fixed to the tensors of the layer, and
 * serving runtimes that size their device memory once at start-up and refuse any
 * allocation afterwards.  For them this entry point runs the persistent stream-K decode
 * kernel (m <= 16) on a scratch array built into the library instead of a caller-owned
 * workspace.  It never allocates: no cudaMalloc, no cudaFree, no allocating library call.
 *
 *   Limit: the built-in scratch is 2 162 688 bytes (64 KiB of row counters plus partial
 *   tiles for 256 CTA ranges of 16 rows).  Layers that need more (aq_linear_workspace_bytes
 *   with AQ_SCHEDULE_AUTO reports the need for layers that take this kernel) are rejected
 *   with AQ_ERR_WORKSPACE; N is limited to 1 048 576.  Every device that loads the library
 *   holds the array until the process exits.
 *   First call on a device: looks up the array's device address (cudaGetSymbolAddress);
 *   make that first call outside of any stream capture.
 *   Sharing: all calls on a device use the same array, and it keeps what the last call
 *   left in it.  Each call clears the row counters it needs on `stream` before the kernel
 *   starts.  Two calls whose kernels may overlap on the GPU (different streams) race on
 *   the array and produce wrong results; serialise them.
 *   Arguments as for aq_linear; the summation order is that of kernel family 2 of
 *   aq_linear_plan (ranges = number of CTAs of that kernel, 16 accumulators).
 */
AQ_API int aq_linear_decode_static(const int8_t* xq, const float* act_scales, int scale_mode,
                                   int64_t m, const void* prepared, int32_t n_j, int32_t n_k,
                                   const int32_t* u_metadata, int out_dtype, void* out, void* stream);

/*
 * How aq_linear will run a problem on the current device, so that a caller can
 * reproduce the FP32 summation order (the integer tile sums never depend on it):
 *   *kernel  0  cluster kernel: K tiles cut into *splits ranges
 *               [n_k*s/splits, n_k*(s+1)/splits), tiles of a range added in increasing k,
 *               range sums added in range order (the reference's split-K order,
 *               alignquant/kernels/cuda/linear.cu:1237-1238, 1339-1343)
 *            1  tensor-memory GEMM: like 0 (K tiles cut into *splits ranges, split sums added in
 *               split order); *splits is 1 unless few rows would leave most SMs idle
 *            2  persistent stream-K kernel: the (j, k)-ordered tile sequence cut into
 *               *splits contiguous ranges [i*T/splits, (i+1)*T/splits); inside a range
 *               tile t goes to accumulator (t - range begin) % *workers
 *            3  warp-per-tile decode kernels: ranges as for 0; inside a range tile k
 *               goes to accumulator (k - range begin) % *workers.  Layers with at least as many
 *               groups of 16 output columns as the GPU has SMs run without a K split
 *               (*splits == 1, register-staged kernel), narrower ones split K over a cluster
 *   In 2 and 3 every accumulator adds its tiles in increasing k, the accumulators of a
 *   range (row segment) are added in index order, and the range sums in range order.
 * The reference's counterpart is its split-K heuristic (linear.cu:1679-1691).
 */
AQ_API int aq_linear_plan(int64_t m, int32_t n_j, int32_t n_k, int schedule, int decode_splits,
                          int32_t* kernel, int32_t* splits, int32_t* workers);

/*
 * Sum of the partial outputs of a row-parallel (K-sharded) projection over the ranks of
 * one node, through peer memory.  The reference has no counterpart: it runs on one GPU and
 * contains no collective.  This stands in for the dist.all_reduce that tensor parallelism
 * needs after o_proj and down_proj, for the small messages of decode; one process per GPU.
 *   Every rank allocates an exchange buffer of aq_allreduce_buffer_bytes(world, max_count)
 *   bytes that all ranks of the node can address (peer-mapped: a CUDA IPC / VMM mapping,
 *   torch symmetric memory ...), zeroes it once, and all ranks synchronise on the host
 *   before the first call.  peer_buffers[r] is rank r's buffer as seen from this process
 *   (a HOST array of `world` device pointers, peer_buffers[rank] being the own one).
 *   partial, out: FP32 [count] in ordinary device memory, 16-byte aligned; count a multiple
 *   of 4, count <= max_count, max_count a multiple of 4; 2 <= world <= 8.  All ranks must
 *   issue the same sequence of calls with the same count and max_count.  The ranks' partials
 *   are added in rank order, so every rank receives the same bits; `out` may alias `partial`.
 *   The call is one asynchronous kernel launch on `stream` (it can be captured and replayed:
 *   the call counter lives in the exchange buffer).  The kernel waits for the peers' data
 *   with a bounded poll (AQ_OPT_PEER_POLL_LIMIT); when a peer never arrives the wait gives up,
 *   the kernel still ends normally, the output is invalid and aq_device_status reports
 *   AQ_ERR_DEVICE naming the rank.  Zero the exchange buffers of all ranks before using them again.
 */
AQ_API int64_t aq_allreduce_buffer_bytes(int32_t world, int64_t max_count);
/*
 * aq_linear followed by that sum, in ONE kernel: the decode kernel's epilogue pushes the
 * finished values of this rank to the peers' exchange buffers and adds the ranks' values in
 * rank order (same protocol, same buffers and call sequence as aq_allreduce_f32; the two may be
 * mixed as long as every rank issues the same sequence).  Automatic schedule only, and only
 * where aq_linear_plan reports kernel 3 (decode sizes, at most 32 rows); otherwise
 * AQ_ERR_INVALID, and the caller uses aq_linear + aq_allreduce_f32.  m * N <= max_count.
 * `out` receives the summed result in out_dtype.  next_prepared / next_bytes: look-ahead as in
 * aq_linear_ahead (NULL / 0: none).
 */
AQ_API int aq_linear_allreduce(const int8_t* xq, const float* act_scales, int scale_mode, int64_t m,
                               const void* prepared, int32_t n_j, int32_t n_k, const int32_t* u_metadata,
                               int out_dtype, void* out, int32_t rank, int32_t world, void* const* peer_buffers,
                               int64_t max_count, const void* next_prepared, int64_t next_bytes, void* stream);
AQ_API int aq_allreduce_f32(const float* partial, float* out, int64_t count, int32_t rank, int32_t world,
                            void* const* peer_buffers, int64_t max_count, void* stream);

/*
 * The per-token activation quantizer and the projection as ONE call, optionally with the sum
 * over the tensor-parallel ranks: what the reference's quantized module does per projection
 * group with two extension calls (alignquant/quantization/model.py:329-350: quantizer, then
 * linear).  Same results, bit for bit, as
 *   aq_quantize_act(x, x_dtype, m, 64 * n_k, NULL, AQ_SCALE_TOKEN, xq, act_scales)  followed by
 *   aq_linear_ahead(xq, act_scales, AQ_SCALE_TOKEN, ...)  or  aq_linear_allreduce(...),
 * and xq / act_scales hold the quantized activations afterwards in either case.  Where the
 * decode kernel of many small CTAs takes the problem and there is ONE row of fp16 / bf16
 * activations (aq_quant_linear_fused returns 1), both run as one launch: every CTA of that kernel
 * reads the whole row anyway, so it finds the row's maximum and rounds the row into its shared
 * memory itself; a launch, its dependency latency and a round trip of the int8 row through the
 * L2 go away.  (The rounding is then repeated on every SM, which at more rows costs more than
 * the launch it saves.)  Everywhere else the call enqueues the quantizer kernel and then the
 * projection.
 *   x            x_dtype [m][64 * n_k] row-major, no input transform (identity V)
 *   xq, act_scales  int8 [m][64 * n_k] and float [m]: outputs (and the projection's operands)
 *   workspace    as for aq_linear (aq_linear_workspace_bytes with the automatic schedule)
 *   peer_buffers NULL: no sum (rank / world / max_count ignored).  Otherwise as for
 *                aq_linear_allreduce, with the same restriction (AQ_ERR_INVALID where
 *                aq_linear_plan does not report kernel 3).
 *   next_prepared / next_bytes  look-ahead as in aq_linear_ahead (NULL / 0: none)
 */
AQ_API int aq_quant_linear(const void* x, int x_dtype, int64_t m, const void* prepared, int32_t n_j, int32_t n_k,
                           const int32_t* u_metadata, int out_dtype, void* out, int8_t* xq, float* act_scales,
                           void* workspace, int64_t workspace_bytes, int32_t rank, int32_t world,
                           void* const* peer_buffers, int64_t max_count, const void* next_prepared,
                           int64_t next_bytes, void* stream);
/* 1 if aq_quant_linear runs this problem (fp16 / bf16 activations) as one launch, else 0. */
AQ_API int aq_quant_linear_fused(int64_t m, int32_t n_j, int32_t n_k);

/*
 * Measurement aid: how fast this GPU's tensor cores execute tcgen05.mma kind::i8 when nothing
 * else happens (operands resident in shared memory, no accumulator drain): one CTA per SM issues
 * `pairs` x 2 MMAs of shape M128 N256 K32 back to back.  Runs the kernel twice on `stream`
 * (warm-up, timed with CUDA events), SYNCHRONISES, and stores integer tera-operations per second
 * in *tops (host pointer).  It is the denominator of the GEMM's tensor-pipe fraction, taken on
 * the same device and clocks.  pairs in [16, 2^20]; 4096 takes about half a millisecond.  The
 * reference has no counterpart.
 */
AQ_API int aq_measure_int8_peak(int32_t pairs, double* tops, void* stream);

/*
 * Synchronises `stream`, then returns AQ_ERR_DEVICE if a kernel of this library gave
 * up a bounded device-side wait since the last call (the outputs of that launch are
 * invalid), clearing the condition; AQ_OK otherwise.  The reference has no such
 * state: its kernels contain no device-side waits.
 */
AQ_API int aq_device_status(void* stream);

#ifdef __cplusplus
}
#endif
#endif /* ALIGNQUANT_B200_H_ */
