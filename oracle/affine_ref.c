/* CPU restatement in plain C of the affine packed-row quantized matmul.  TEST INFRASTRUCTURE: the checker for sizes
 * numpy is too slow for, and the timed host baseline of bench.py.  Never linked into the product library.
 *
 * Format and arithmetic follow the reference project:
 *   code extraction    cuda/kernels/affine_kernels.py:7-14, kernels/qwen/dense/v1/affine_rows.py:14-21
 *   dequantisation     families/qwen3_5/cuda/qmm.py:132-149   (w = q * scale + bias, float32)
 *   matmul             tests/cuda/test_qmm.py:22-26,64-70     (x.float() @ w.T)
 */
#include <math.h>
#ifdef _OPENMP
#include <omp.h>
#endif
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

static inline float bf16_to_f32(uint16_t v) {
  uint32_t u = (uint32_t)v << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}

static inline uint32_t code_of(const uint32_t* row, int64_t k, int bits, int64_t words) {
  const int64_t bit = k * bits, word = bit >> 5;
  const int shift = (int)(bit & 31);
  uint64_t v = row[word];
  if (shift + bits > 32 && word + 1 < words) v |= (uint64_t)row[word + 1] << 32;
  return (uint32_t)((v >> shift) & ((1u << bits) - 1u));
}

/* w_out[n, k] (float32) = q * scale + bias; scales/biases are bf16 bit patterns [n, k/gs]. */
void oracle_dequantize(const uint32_t* words, const uint16_t* scales, const uint16_t* biases, int64_t n, int64_t k,
                       int bits, int gs, float* w_out) {
  const int64_t wpr = k * bits / 32, kg = k / gs;
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < n; ++r) {
    const uint32_t* row = words + r * wpr;
    for (int64_t c = 0; c < k; ++c) {
      const float s = bf16_to_f32(scales[r * kg + c / gs]), b = bf16_to_f32(biases[r * kg + c / gs]);
      w_out[r * k + c] = (float)code_of(row, c, bits, wpr) * s + b;
    }
  }
}

/* out[m, n] (double) = sum_k x[m, k] * (q[n, k] * s + b); x is bf16 bit patterns [m, k]. Dequantises on the fly. */
void oracle_qmm_f64(const uint16_t* x, int64_t m, const uint32_t* words, const uint16_t* scales, const uint16_t* biases,
                    int64_t n, int64_t k, int bits, int gs, double* out) {
  const int64_t wpr = k * bits / 32, kg = k / gs;
#pragma omp parallel
  {
    double* w = (double*)malloc(sizeof(double) * (size_t)k);
#pragma omp for schedule(static)
    for (int64_t r = 0; r < n; ++r) {
      const uint32_t* row = words + r * wpr;
      for (int64_t c = 0; c < k; ++c) {
        const double s = bf16_to_f32(scales[r * kg + c / gs]), b = bf16_to_f32(biases[r * kg + c / gs]);
        w[c] = (double)code_of(row, c, bits, wpr) * s + b;
      }
      for (int64_t i = 0; i < m; ++i) {
        double acc = 0.0;
        const uint16_t* xr = x + i * k;
        for (int64_t c = 0; c < k; ++c) acc += (double)bf16_to_f32(xr[c]) * w[c];
        out[i * n + r] = acc;
      }
    }
    free(w);
  }
}

/* Same in float32 (dequantise a row to float32, then a float32 dot): the host-baseline flavour. */
void oracle_qmm_f32(const uint16_t* x, int64_t m, const uint32_t* words, const uint16_t* scales, const uint16_t* biases,
                    int64_t n, int64_t k, int bits, int gs, float* out) {
  const int64_t wpr = k * bits / 32, kg = k / gs;
#pragma omp parallel
  {
    float* w = (float*)malloc(sizeof(float) * (size_t)k);
    float* xf = (float*)malloc(sizeof(float) * (size_t)k);
#pragma omp for schedule(static)
    for (int64_t r = 0; r < n; ++r) {
      const uint32_t* row = words + r * wpr;
      for (int64_t c = 0; c < k; ++c) {
        const float s = bf16_to_f32(scales[r * kg + c / gs]), b = bf16_to_f32(biases[r * kg + c / gs]);
        w[c] = (float)code_of(row, c, bits, wpr) * s + b;
      }
      for (int64_t i = 0; i < m; ++i) {
        const uint16_t* xr = x + i * k;
        for (int64_t c = 0; c < k; ++c) xf[c] = bf16_to_f32(xr[c]);
        float acc = 0.f;
        for (int64_t c = 0; c < k; ++c) acc += xf[c] * w[c];
        out[i * n + r] = acc;
      }
    }
    free(w);
    free(xf);
  }
}

int oracle_threads(void) {
  int t = 1;
#ifdef _OPENMP
#pragma omp parallel
  {
#pragma omp master
    t = omp_get_num_threads();
  }
#endif
  return t;
}

/* Threads the parallel loops use from now on (a launcher may have exported OMP_NUM_THREADS=1 for its workers). */
void oracle_set_threads(int n) {
  if (n > 0) omp_set_num_threads(n);
}
