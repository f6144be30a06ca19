/*
 * CPU oracle, compiled form (TEST INFRASTRUCTURE ONLY; see oracle/__init__.py).
 *
 * Restates the reference's quantised gather-matmul arithmetic in plain C so
 * that parity cases larger than NumPy handles comfortably, and the host-CPU
 * timing printed beside the GPU number, finish in seconds.  Nothing in the
 * shipped package links or loads this file.
 *
 * Arithmetic followed (reference paths are relative to the ZMLX tree):
 *   - packed layout and affine dequantisation: src/zmlx/kernels/quant.py:109-120
 *     (code i of a row is (word[i/8] >> 4*(i%8)) & 0xF; w = q*scale + bias;
 *     float32 accumulation of w*x);
 *   - fused gate/up + SwiGLU, CPU contract:
 *     integrations/mlx_local_integration/gather_qmm_swiglu.patch:47-55, 142-186
 *     (both projections materialised in T, then g * 1/(1+exp(-g)) * u in float,
 *     rounded once);
 *   - mxfp4: OCP microscaling e2m1 codes, one e8m0 scale per 32 (the reference
 *     has no mxfp4 arithmetic of its own).  Parity unpinned.
 *
 * Build: see oracle/Makefile (gcc -O3 -fopenmp -shared -fPIC).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

static inline float bf16_to_f32(uint16_t h) {
  uint32_t u = ((uint32_t)h) << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}

static inline uint16_t f32_to_bf16(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)((u >> 16) | 0x0040u); /* NaN */
  u += 0x7FFFu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}

static const float kE2M1[16] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f,
                                -0.0f, -0.5f, -1.0f, -1.5f, -2.0f, -3.0f, -4.0f, -6.0f};

int zo_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

void zo_set_num_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

/* One output row-dot, affine 4-bit: sum_k x[k] * (q[k]*s[k/gs] + b[k/gs]). */
static inline float dot_affine(const float* x, const uint32_t* w, const uint16_t* s, const uint16_t* b,
                               int K, int gs) {
  float acc = 0.0f;
  const int ngroups = K / gs;
  for (int g = 0; g < ngroups; ++g) {
    const float sc = bf16_to_f32(s[g]);
    const float bi = bf16_to_f32(b[g]);
    const uint32_t* wg = w + (size_t)g * (gs / 8);
    const float* xg = x + (size_t)g * gs;
    float part = 0.0f;
#pragma omp simd reduction(+ : part)
    for (int i = 0; i < gs; ++i) {
      const uint32_t q = (wg[i >> 3] >> (4 * (i & 7))) & 0xFu;
      part += ((float)q * sc + bi) * xg[i];
    }
    acc += part;
  }
  return acc;
}

static inline float dot_mxfp4(const float* x, const uint32_t* w, const uint8_t* s, int K) {
  float acc = 0.0f;
  const int ngroups = K / 32;
  for (int g = 0; g < ngroups; ++g) {
    const float sc = ldexpf(1.0f, (int)s[g] - 127);
    const uint32_t* wg = w + (size_t)g * 4;
    const float* xg = x + (size_t)g * 32;
    float part = 0.0f;
    for (int i = 0; i < 32; ++i) {
      const uint32_t q = (wg[i >> 3] >> (4 * (i & 7))) & 0xFu;
      part += (kE2M1[q] * sc) * xg[i];
    }
    acc += part;
  }
  return acc;
}

/*
 * out[p, :] = T( x[lhs[p], :] @ dequant(W[rhs[p]]).T ), p in [0, P).
 * x: (R, K) bf16 bits; w: (E, N, K/8); mode 0 = affine (scales/biases (E, N, K/gs) bf16),
 * mode 1 = mxfp4 (scales (E, N, K/32) uint8, biases ignored).  Returns 0, or -1 on a bad index.
 */
int zo_gather_qmm(const uint16_t* x, int R, const uint32_t* w, const void* scales, const uint16_t* biases,
                  int E, int N, int K, int gs, int mode, const int32_t* lhs, const int32_t* rhs, int P,
                  uint16_t* out) {
  for (int p = 0; p < P; ++p)
    if (lhs[p] < 0 || lhs[p] >= R || rhs[p] < 0 || rhs[p] >= E) return -1;
  const int G = (mode == 0) ? K / gs : K / 32;
  const int total = P * N;
#pragma omp parallel
  {
    float* xf = (float*)malloc(sizeof(float) * (size_t)K);
    int cached = -1;
#pragma omp for schedule(static)
    for (int i = 0; i < total; ++i) {
      const int p = i / N, n = i % N;
      if (cached != lhs[p]) {
        const uint16_t* xr = x + (size_t)lhs[p] * K;
        for (int k = 0; k < K; ++k) xf[k] = bf16_to_f32(xr[k]);
        cached = lhs[p];
      }
      const size_t row = (size_t)rhs[p] * N + n;
      const uint32_t* wr = w + row * (size_t)(K / 8);
      float v;
      if (mode == 0)
        v = dot_affine(xf, wr, (const uint16_t*)scales + row * G, biases + row * G, K, gs);
      else
        v = dot_mxfp4(xf, wr, (const uint8_t*)scales + row * G, K);
      out[(size_t)p * N + n] = f32_to_bf16(v);
    }
    free(xf);
  }
  return 0;
}

/* contract 0: T(g * 1/(1+exp(-g)) * u) in float (CPU contract of the fused op). */
void zo_swiglu(const uint16_t* g, const uint16_t* u, uint16_t* out, long n) {
#pragma omp parallel for schedule(static)
  for (long i = 0; i < n; ++i) {
    const float gf = bf16_to_f32(g[i]);
    const float uf = bf16_to_f32(u[i]);
    const float sig = 1.0f / (1.0f + expf(-gf));
    out[i] = f32_to_bf16(gf * sig * uf);
  }
}

/*
 * Ordered weighted combine over K slots: out[t, d] = sum_i w[t,i] * y[t,i,d], the
 * product rounded to float32 before the add (no contraction), float32 result.
 * src/zmlx/kernels/moe.py:1075-1095.
 */
void zo_combine_fp32_no_fma(const uint16_t* y, const float* w, int T, int K, int D, float* out) {
#pragma omp parallel for schedule(static)
  for (int t = 0; t < T; ++t) {
    for (int d = 0; d < D; ++d) {
      volatile float acc = 0.0f;
      for (int i = 0; i < K; ++i) {
        volatile float prod = w[t * K + i] * bf16_to_f32(y[((size_t)t * K + i) * D + d]);
        acc = acc + prod;
      }
      out[(size_t)t * D + d] = acc;
    }
  }
}
