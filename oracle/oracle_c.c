/*
 * CPU restatement, in plain C with OpenMP, of the hot-path ops the benchmarks time.
 *
 * TEST INFRASTRUCTURE ONLY: used as the parity checker's fast twin (pinned
 * against oracle.py in the CPU tests) and as the timed CPU baseline in bench.py
 * ("cpu_baseline" and "--impl reference").  Nothing in the product links it.
 *
 * The reference (gomlx/go-darwinml) has no CPU implementation of these ops --
 * each is one call into Apple's closed MPSGraph framework -- so this follows the
 * formulas its Go lowering spells out:
 *   softmax        max-subtracted form, last axis       (mpsgraph bridge.m:1448-1461; test mpsgraph_test.go:1182-1189)
 *   causal mask    keep column j of row i iff i >= j    (mpsgraph function.go:2777-2794)
 *   LayerNorm      two-pass biased variance, rsqrt      (mpsgraph function.go:2430-2558)
 *   RMSNorm        x * rsqrt(mean(x^2)+eps) * gamma     (absent from the reference; defined here)
 *   DotGeneral     [B,M,K] x [B,K,N] or [B,K,M] x [B,K,N], fp32 accumulate (mpsgraph dotgeneral.go:65-164)
 * Timed path: float32 arithmetic.  bf16 values are stored as uint16_t.
 *
 * Build: gcc -O3 -march=native -fopenmp -shared -fPIC oracle_c.c -o liboracle_c.so -lm
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

static inline float bf16_to_f32(uint16_t h) {
  uint32_t u = (uint32_t)h << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}
static inline uint16_t f32_to_bf16(float f) { /* round to nearest even */
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40);
  u += 0x7fffu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}

/* y[r, :] = softmax(scale * x[r, :]) with columns j > (r % seq_q) masked to -inf when causal != 0. */
void oracle_softmax_f32(const float* x, float* y, int64_t rows, int64_t cols, float scale, int causal, int64_t seq_q) {
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < rows; ++r) {
    const float* xr = x + r * cols;
    float* yr = y + r * cols;
    int64_t limit = cols;
    if (causal) {
      int64_t q = r % seq_q;
      limit = q + 1 < cols ? q + 1 : cols;
    }
    float mx = -INFINITY;
    for (int64_t j = 0; j < limit; ++j) {
      float s = xr[j] * scale;
      mx = s > mx ? s : mx;
    }
    float sum = 0.f;
    for (int64_t j = 0; j < limit; ++j) {
      float e = expf(xr[j] * scale - mx);
      yr[j] = e;
      sum += e;
    }
    float inv = 1.0f / sum;
    for (int64_t j = 0; j < limit; ++j) yr[j] *= inv;
    for (int64_t j = limit; j < cols; ++j) yr[j] = 0.f;
  }
}

/* rms != 0: RMSNorm (beta ignored); else LayerNorm.  gamma / beta may be NULL. */
void oracle_norm_bf16(const uint16_t* x, const uint16_t* gamma, const uint16_t* beta, uint16_t* y, int64_t rows, int64_t cols,
                      float eps, int rms) {
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < rows; ++r) {
    const uint16_t* xr = x + r * cols;
    uint16_t* yr = y + r * cols;
    float mean = 0.f;
    if (!rms) {
      float s = 0.f;
      for (int64_t j = 0; j < cols; ++j) s += bf16_to_f32(xr[j]);
      mean = s / (float)cols;
    }
    float sq = 0.f;
    for (int64_t j = 0; j < cols; ++j) {
      float d = bf16_to_f32(xr[j]) - mean;
      sq += d * d;
    }
    float rstd = 1.0f / sqrtf(sq / (float)cols + eps);
    for (int64_t j = 0; j < cols; ++j) {
      float v = (bf16_to_f32(xr[j]) - mean) * rstd;
      if (gamma) v *= bf16_to_f32(gamma[j]);
      if (!rms && beta) v += bf16_to_f32(beta[j]);
      yr[j] = f32_to_bf16(v);
    }
  }
}

void oracle_norm_f32(const float* x, const float* gamma, const float* beta, float* y, int64_t rows, int64_t cols, float eps, int rms) {
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < rows; ++r) {
    const float* xr = x + r * cols;
    float* yr = y + r * cols;
    double mean = 0.0;
    if (!rms) {
      double s = 0.0;
      for (int64_t j = 0; j < cols; ++j) s += xr[j];
      mean = s / (double)cols;
    }
    double sq = 0.0;
    for (int64_t j = 0; j < cols; ++j) {
      double d = xr[j] - mean;
      sq += d * d;
    }
    double rstd = 1.0 / sqrt(sq / (double)cols + (double)eps);
    for (int64_t j = 0; j < cols; ++j) {
      double v = (xr[j] - mean) * rstd;
      if (gamma) v *= gamma[j];
      if (!rms && beta) v += beta[j];
      yr[j] = (float)v;
    }
  }
}

/* C[b,m,n] = sum_k A(b,m,k) * B(b,k,n); a_k_major: A is [B,M,K] else [B,K,M]; b_k_major: B is [B,N,K] else [B,K,N].
 * fp32 inputs, fp32 accumulation, blocked over k for cache reuse. */
void oracle_gemm_f32(const float* a, const float* b, float* c, int64_t batch, int64_t m, int64_t n, int64_t k, int a_k_major,
                     int b_k_major) {
  const int64_t a_sm = a_k_major ? k : 1, a_sk = a_k_major ? 1 : m;
  const int64_t b_sk = b_k_major ? 1 : n, b_sn = b_k_major ? k : 1;
#pragma omp parallel for collapse(2) schedule(static)
  for (int64_t bi = 0; bi < batch; ++bi) {
    for (int64_t i = 0; i < m; ++i) {
      const float* ab = a + bi * m * k;
      const float* bb = b + bi * k * n;
      float* cr = c + (bi * m + i) * n;
      for (int64_t j = 0; j < n; ++j) cr[j] = 0.f;
      if (!b_k_major) {
        for (int64_t kk = 0; kk < k; ++kk) {
          const float av = ab[i * a_sm + kk * a_sk];
          const float* br = bb + kk * n;
          for (int64_t j = 0; j < n; ++j) cr[j] += av * br[j];
        }
      } else {
        for (int64_t j = 0; j < n; ++j) {
          float acc = 0.f;
          for (int64_t kk = 0; kk < k; ++kk) acc += ab[i * a_sm + kk * a_sk] * bb[kk * b_sk + j * b_sn];
          cr[j] = acc;
        }
      }
    }
  }
}

/* Same with bf16 storage (uint16_t), fp32 accumulation, one final rounding. */
void oracle_gemm_bf16(const uint16_t* a, const uint16_t* b, uint16_t* c, int64_t batch, int64_t m, int64_t n, int64_t k,
                      int a_k_major, int b_k_major) {
  const int64_t a_sm = a_k_major ? k : 1, a_sk = a_k_major ? 1 : m;
  const int64_t b_sk = b_k_major ? 1 : n, b_sn = b_k_major ? k : 1;
#pragma omp parallel for collapse(2) schedule(static)
  for (int64_t bi = 0; bi < batch; ++bi) {
    for (int64_t i = 0; i < m; ++i) {
      const uint16_t* ab = a + bi * m * k;
      const uint16_t* bb = b + bi * k * n;
      float* acc = (float*)calloc((size_t)n, sizeof(float));
      for (int64_t kk = 0; kk < k; ++kk) {
        const float av = bf16_to_f32(ab[i * a_sm + kk * a_sk]);
        for (int64_t j = 0; j < n; ++j) acc[j] += av * bf16_to_f32(bb[kk * b_sk + j * b_sn]);
      }
      for (int64_t j = 0; j < n; ++j) c[(bi * m + i) * n + j] = f32_to_bf16(acc[j]);
      free(acc);
    }
  }
}

/* Sets the OpenMP team size for the calls that follow (launchers such as torchrun export OMP_NUM_THREADS=1). */
void oracle_set_num_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

int oracle_num_threads(void) {
  int n = 1;
#ifdef _OPENMP
#pragma omp parallel
  {
#pragma omp master
    n = omp_get_num_threads();
  }
#endif
  return n;
}
