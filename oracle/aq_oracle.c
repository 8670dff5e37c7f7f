/*
 * C restatement of the integer core of the AlignQuant mixed W4/W8-A8 linear
 * layer.  TEST INFRASTRUCTURE ONLY: it is the checker for the CUDA kernels and
 * the timed CPU baseline of the benchmark; the shipped library never links it.
 *
 * Inputs are the *logical* operands: int8 activations xq[M][K], float32
 * activation scales a[M][n_k] (already broadcast per row), int8 weight tiles
 * w[n_j][n_k][64 out][64 in] (W4 tiles hold values in [-8, 7]) and float32 tile
 * scales ws[n_j][n_k].  The arithmetic follows the reference kernels:
 *   - per (row, N64 tile, K64 tile) exact int32 dot product of 64 terms
 *     (alignquant/kernels/cuda/linear.cu:664-686, 941-950);
 *   - FP32 path: acc = acc + float(int) * (a * ws), float multiply and add
 *     rounded separately, K tiles in increasing order, split-K planes summed in
 *     split order (linear.cu:956-963, 1237-1238, 1296-1301, 1339-1343);
 *   - FP64 path: the reference's CPU dequantize-and-matmul
 *     (alignquant/quantization/exact.py:277-285 and
 *     alignquant/quantization/calibration.py:566-567), identity output transform.
 *
 *   - fused FP32 variant (fused != 0): acc = fma(float(int), a * ws, acc), one rounding
 *     per tile instead of two -- the order of the tensor-memory GEMM's default drain.
 *
 * Build: gcc -O3 -march=x86-64-v3 -ffp-contract=off -fopenmp -shared -fPIC aq_oracle.c -o libaq_oracle.so -lm
 * (-ffp-contract=off keeps every multiply and add separately rounded, as the
 * FP32 contract requires; the fused variant calls fmaf explicitly.)
 */
#include <math.h>
#include <stdint.h>
#include <stddef.h>

#define TILE 64

static inline int32_t dot64(const int8_t* a, const int8_t* b) {
  int32_t s = 0;
  for (int i = 0; i < TILE; ++i) s += (int32_t)a[i] * (int32_t)b[i];
  return s;
}

/* out[M][n_j][n_k][64] */
void aqo_tile_accumulators(const int8_t* xq, const int8_t* w, int32_t* out,
                           int64_t M, int64_t n_j, int64_t n_k) {
#pragma omp parallel for collapse(2) schedule(static)
  for (int64_t m = 0; m < M; ++m) {
    for (int64_t j = 0; j < n_j; ++j) {
      for (int64_t k = 0; k < n_k; ++k) {
        const int8_t* a = xq + (m * n_k + k) * TILE;
        const int8_t* t = w + ((j * n_k + k) * TILE) * TILE;
        int32_t* o = out + ((m * n_j + j) * n_k + k) * TILE;
        for (int c = 0; c < TILE; ++c) o[c] = dot64(a, t + c * TILE);
      }
    }
  }
}

/*
 * out[M][n_j*64] float32, kernel operation order.  K tiles are cut into split_k ranges
 * [n_k*s/split_k, n_k*(s+1)/split_k); inside a range tile k belongs to worker
 * (k - range_begin) % workers, every worker adds its tiles in increasing k, the worker
 * sums are added in worker order and the range sums in range order.  workers = 1 is the
 * reference kernels' own order.
 */
static void linear_fp32_impl(const int8_t* xq, const float* a, const int8_t* w, const float* ws,
                             float* out, int64_t M, int64_t n_j, int64_t n_k, int64_t split_k, int64_t workers,
                             int fused) {
  if (split_k < 1) split_k = 1;
  if (workers < 1) workers = 1;
  if (workers > 64) workers = 64;
#pragma omp parallel for collapse(2) schedule(static)
  for (int64_t j = 0; j < n_j; ++j) {
    for (int64_t m = 0; m < M; ++m) {
      float total[TILE];
      for (int64_t s = 0; s < split_k; ++s) {
        float part[64][TILE];
        for (int64_t v = 0; v < workers; ++v)
          for (int c = 0; c < TILE; ++c) part[v][c] = 0.0f;
        const int64_t k0 = n_k * s / split_k, k1 = n_k * (s + 1) / split_k;
        for (int64_t k = k0; k < k1; ++k) {
          const int64_t v = (k - k0) % workers;
          const float scale = a[m * n_k + k] * ws[j * n_k + k];
          const int8_t* x = xq + (m * n_k + k) * TILE;
          const int8_t* t = w + ((j * n_k + k) * TILE) * TILE;
          if (fused) {
            for (int c = 0; c < TILE; ++c) part[v][c] = fmaf((float)dot64(x, t + c * TILE), scale, part[v][c]);
          } else {
            for (int c = 0; c < TILE; ++c) {
              const float scaled = (float)dot64(x, t + c * TILE) * scale;
              part[v][c] = part[v][c] + scaled;
            }
          }
        }
        for (int c = 0; c < TILE; ++c) {
          float seg = part[0][c];
          for (int64_t v = 1; v < workers; ++v) seg = seg + part[v][c];
          total[c] = (s == 0) ? seg : total[c] + seg;
        }
      }
      for (int c = 0; c < TILE; ++c) out[m * n_j * TILE + j * TILE + c] = total[c];
    }
  }
}

void aqo_linear_fp32(const int8_t* xq, const float* a, const int8_t* w, const float* ws,
                     float* out, int64_t M, int64_t n_j, int64_t n_k, int64_t split_k, int64_t workers) {
  linear_fp32_impl(xq, a, w, ws, out, M, n_j, n_k, split_k, workers, 0);
}

/* acc = fma(float(int), a * ws, acc): the product a * ws is still rounded to FP32 first. */
void aqo_linear_fp32_fused(const int8_t* xq, const float* a, const int8_t* w, const float* ws,
                           float* out, int64_t M, int64_t n_j, int64_t n_k, int64_t split_k, int64_t workers) {
  linear_fp32_impl(xq, a, w, ws, out, M, n_j, n_k, split_k, workers, 1);
}

/*
 * Same arithmetic as aqo_linear_fp32 with the sums grouped the way the persistent
 * decode kernel groups them.  The (j, k)-ordered tile sequence of T = n_j*n_k tiles is
 * split into `ranges` contiguous ranges, range i = [i*T/ranges, (i+1)*T/ranges).
 * Inside a range, tile t belongs to worker (t - range_begin) % workers; for every row
 * segment of the range each worker adds its tiles in increasing k, the worker sums are
 * added in worker order, and the segment sums of the ranges sharing a row are added in
 * range order.
 */
void aqo_linear_fp32_ranges(const int8_t* xq, const float* a, const int8_t* w, const float* ws,
                            float* out, int64_t M, int64_t n_j, int64_t n_k, int64_t ranges,
                            int64_t workers) {
  const int64_t T = n_j * n_k;
  if (ranges < 1) ranges = 1;
  if (ranges > T) ranges = T;
  if (workers < 1) workers = 1;
  if (workers > 64) workers = 64;
#pragma omp parallel for collapse(2) schedule(static)
  for (int64_t j = 0; j < n_j; ++j) {
    for (int64_t m = 0; m < M; ++m) {
      float total[TILE];
      int first = 1;
      int64_t k = 0;
      while (k < n_k) {
        const int64_t t = j * n_k + k;
        const int64_t owner = ((t + 1) * ranges - 1) / T;
        const int64_t begin = owner * T / ranges;
        int64_t end = (owner + 1) * T / ranges - j * n_k; /* first k of the next range */
        if (end > n_k) end = n_k;
        float part[64][TILE];
        for (int64_t v = 0; v < workers; ++v)
          for (int c = 0; c < TILE; ++c) part[v][c] = 0.0f;
        for (; k < end; ++k) {
          const int64_t v = (j * n_k + k - begin) % workers;
          const float scale = a[m * n_k + k] * ws[j * n_k + k];
          const int8_t* x = xq + (m * n_k + k) * TILE;
          const int8_t* tl = w + ((j * n_k + k) * TILE) * TILE;
          for (int c = 0; c < TILE; ++c) {
            const float scaled = (float)dot64(x, tl + c * TILE) * scale;
            part[v][c] = part[v][c] + scaled;
          }
        }
        for (int c = 0; c < TILE; ++c) {
          float seg = part[0][c];
          for (int64_t v = 1; v < workers; ++v) seg = seg + part[v][c];
          total[c] = first ? seg : total[c] + seg;
        }
        first = 0;
      }
      for (int c = 0; c < TILE; ++c) out[m * n_j * TILE + j * TILE + c] = total[c];
    }
  }
}

/* out[M][n_j*64] float64: sum_k (xq*a) . (w*ws), all products and sums in FP64 */
void aqo_linear_fp64(const int8_t* xq, const float* a, const int8_t* w, const float* ws,
                     double* out, int64_t M, int64_t n_j, int64_t n_k) {
#pragma omp parallel for collapse(2) schedule(static)
  for (int64_t j = 0; j < n_j; ++j) {
    for (int64_t m = 0; m < M; ++m) {
      double acc[TILE];
      for (int c = 0; c < TILE; ++c) acc[c] = 0.0;
      for (int64_t k = 0; k < n_k; ++k) {
        const double sa = (double)a[m * n_k + k];
        const double sw = (double)ws[j * n_k + k];
        const int8_t* x = xq + (m * n_k + k) * TILE;
        const int8_t* t = w + ((j * n_k + k) * TILE) * TILE;
        for (int c = 0; c < TILE; ++c) {
          double s = 0.0;
          for (int i = 0; i < TILE; ++i) s += ((double)x[i] * sa) * ((double)t[c * TILE + i] * sw);
          acc[c] += s;
        }
      }
      for (int c = 0; c < TILE; ++c) out[m * n_j * TILE + j * TILE + c] = acc[c];
    }
  }
}
