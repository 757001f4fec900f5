/*
 * CPU oracle for the LQQ W4A8 linear path, plain C.  TEST INFRASTRUCTURE ONLY: it is the checker
 * used by the test-suite / smoke run and the timed CPU baseline of the benchmark, never a code
 * path of the product.
 *
 * Parity status: pinned -- tests/test_oracle_c.py compares every function with the numpy oracle
 * (oracle/lqq_oracle.py), which is itself pinned to fixtures computed by the reference.
 *
 * The arithmetic restated here:
 *   q_hat[n,k] = ((code[n,k] * step[n,g] + a[n,g]) XOR 0x80) as int8     liquidgemm/quant.py:103-112
 *   acc[m,n]   = sum_k x[m,k] * q_hat[n,k]              (exact int32)     liquidgemm/quant.py:151
 *   y[m,n]     = (float)acc * ascale[m] * s1[n]         (fp32, in order)  liquidgemm/quant.py:152
 *   per-token activation quantiser                                         liquidgemm/quant.py:135-141
 * OpenMP parallelises over output channels; build with -fopenmp to use every host core.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

/* Pin the team size (a launcher such as torchrun exports OMP_NUM_THREADS=1; the baseline should use the host). */
void lqo_set_num_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

int lqo_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/* codes: [N,K] one 4-bit code per byte.  out: [N,K] int8. */
void lqo_dequant_i8(const uint8_t* codes, const uint8_t* step, const uint8_t* off, int8_t* out,
                    int N, int K, int group) {
  const int G = K / group;
#pragma omp parallel for schedule(static)
  for (int n = 0; n < N; ++n) {
    for (int k = 0; k < K; ++k) {
      const int g = k / group;
      const unsigned u = (unsigned)codes[(size_t)n * K + k] * step[(size_t)n * G + g] + off[(size_t)n * G + g];
      out[(size_t)n * K + k] = (int8_t)((u & 0xFFu) ^ 0x80u);
    }
  }
}

/* Same reconstruction on 32-bit words, four codes per multiply-add (liquidgemm/pack.py:55-78). */
void lqo_dequant_i8_simd(const uint8_t* codes, const uint8_t* step, const uint8_t* off, int8_t* out,
                         int N, int K, int group) {
  const int G = K / group;
#pragma omp parallel for schedule(static)
  for (int n = 0; n < N; ++n) {
    for (int k = 0; k < K; k += 4) {
      const int g = k / group;
      uint32_t w;
      memcpy(&w, codes + (size_t)n * K + k, 4);
      w = (w * (uint32_t)step[(size_t)n * G + g] + (uint32_t)off[(size_t)n * G + g] * 0x01010101u) ^ 0x80808080u;
      memcpy(out + (size_t)n * K + k, &w, 4);
    }
  }
}

/* x: [M,K] int8, qhat: [N,K] int8 -> acc [M,N] int32. */
void lqo_int_gemm(const int8_t* x, const int8_t* qhat, int32_t* acc, int M, int N, int K) {
#pragma omp parallel for schedule(static)
  for (int n = 0; n < N; ++n) {
    const int8_t* w = qhat + (size_t)n * K;
    for (int m = 0; m < M; ++m) {
      const int8_t* xr = x + (size_t)m * K;
      int32_t s = 0;
      for (int k = 0; k < K; ++k) s += (int32_t)xr[k] * (int32_t)w[k];
      acc[(size_t)m * N + n] = s;
    }
  }
}

/* y = (float)acc * ascale[m] * s1[n], left to right. */
void lqo_scale_f32(const int32_t* acc, const float* ascale, const float* s1, float* y, int M, int N) {
#pragma omp parallel for schedule(static)
  for (int m = 0; m < M; ++m) {
    for (int n = 0; n < N; ++n) {
      volatile float t = (float)acc[(size_t)m * N + n] * ascale[m];
      y[(size_t)m * N + n] = t * s1[n];
    }
  }
}

/* Per-token symmetric INT8: scale = max(amax, 1e-12) / 127, q = clamp(rint(x / scale), +-127). */
void lqo_quant_per_token(const float* x, int8_t* xq, float* ascale, int M, int K) {
#pragma omp parallel for schedule(static)
  for (int m = 0; m < M; ++m) {
    const float* xr = x + (size_t)m * K;
    float amax = 0.f;
    for (int k = 0; k < K; ++k) {
      const float a = fabsf(xr[k]);
      if (a > amax) amax = a;
    }
    const float sc = (amax > 1e-12f ? amax : 1e-12f) / 127.0f;
    ascale[m] = sc;
    for (int k = 0; k < K; ++k) {
      float q = nearbyintf(xr[k] / sc); /* default rounding mode: to nearest even */
      if (q > 127.f) q = 127.f;
      if (q < -127.f) q = -127.f;
      xq[(size_t)m * K + k] = (int8_t)q;
    }
  }
}

/* The whole linear for one batch of tokens: quantise tokens, dequantise weights on the fly,
 * integer GEMM, scale.  fp32 output [M,N].  This is the timed CPU baseline. */
void lqo_w4a8_linear(const float* x, const uint8_t* codes, const uint8_t* step, const uint8_t* off,
                     const float* s1, float* y, int M, int N, int K, int group) {
  int8_t* xq = (int8_t*)malloc((size_t)M * K);
  float* ascale = (float*)malloc(sizeof(float) * (size_t)M);
  lqo_quant_per_token(x, xq, ascale, M, K);
  const int G = K / group;
#pragma omp parallel
  {
    int8_t* w = (int8_t*)malloc((size_t)K);
#pragma omp for schedule(static)
    for (int n = 0; n < N; ++n) {
      for (int k = 0; k < K; k += 4) {
        const int g = k / group;
        uint32_t v;
        memcpy(&v, codes + (size_t)n * K + k, 4);
        v = (v * (uint32_t)step[(size_t)n * G + g] + (uint32_t)off[(size_t)n * G + g] * 0x01010101u) ^ 0x80808080u;
        memcpy(w + k, &v, 4);
      }
      for (int m = 0; m < M; ++m) {
        const int8_t* xr = xq + (size_t)m * K;
        int32_t s = 0;
        for (int k = 0; k < K; ++k) s += (int32_t)xr[k] * (int32_t)w[k];
        volatile float t = (float)s * ascale[m];
        y[(size_t)m * N + n] = t * s1[n];
      }
    }
    free(w);
  }
  free(xq);
  free(ascale);
}
