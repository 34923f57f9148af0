/*
 * CPU oracle for the q4f16 dequantize + matmul path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file restates, in plain C, the arithmetic that the reference (tlc-pack/relax)
 * produces for a group-quantized matmul once its generic passes have lowered it to
 * TIR and LLVM has compiled that TIR for the CPU.  Nothing here is shipped or
 * measured as the product: only the tests, the smoke check and the CPU-baseline leg
 * of the benchmark may load it.
 *
 * Parity status: the reference holds no golden vectors for int4 decode or grouped
 * scales, and it cannot be built in this environment (no LLVM, empty submodules),
 * so parity with the reference proper is UNPINNED.  The restatement is pinned
 * instead against (1) a third-party descendant of the reference (TVM 0.23 Relax VM,
 * target "c") whose outputs are committed under tests/golden/, and (2) the matmul
 * accumulate semantics that the reference's own legalization test fixes.
 *
 * Semantics followed (paths are relative to the reference tree):
 *   decode   q[n,k] = (Wq[n,k/8] >> 4*(k%8)) & 0xF            src/tir/op/op.cc:564 (right_shift), :606 (bitwise_and)
 *            w[n,k] = fp16(q-7) *fp16 S[n,k/32]               src/tir/op/op.cc:282 (cast); one IEEE RN-even fp16 multiply
 *   matmul   acc[m,n] = sum_k f32(x[m,k]) * f32(w[n,k])       python/tvm/relax/transform/legalize_ops.py:203-264
 *            fp32, k ascending, initial value 0               tests/python/relax/test_transform_legalize_ops_index_linear_algebra.py:283-315
 *   astype   y[m,n] = fp16_rn_even(acc[m,n])                  python/tvm/relax/transform/legalize_ops.py:157-162,
 *                                                             3rdparty/compiler-rt/builtin_fp16.h:111-160
 *
 * (q-7) lies in [-7, 8] and a scale has an 11-bit significand, so the product
 * (q-7)*s is exact in fp32; rounding that fp32 value once to fp16 is therefore the
 * same as a single fp16 multiply.  Likewise f32(x)*f32(w) is exact in fp32, so a
 * fused multiply-add and a separate multiply and add give identical sums.
 *
 * Build: see oracle/Makefile (gcc -O3 -mavx2 -mf16c -fopenmp, no fast-math).
 */
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

typedef _Float16 f16;

static inline float h2f(uint16_t h) {
  f16 v;
  memcpy(&v, &h, 2);
  return (float)v;
}
static inline uint16_t f2h(float f) {
  f16 v = (f16)f; /* round-to-nearest-even */
  uint16_t h;
  memcpy(&h, &v, 2);
  return h;
}

/* Decode one row of packed weights into fp16 bit patterns (w_row has K entries). */
static void decode_row(const uint32_t* wq_row, const uint16_t* s_row, uint16_t* w_row, int64_t K) {
  for (int64_t k = 0; k < K; ++k) {
    uint32_t word = wq_row[k >> 3];
    int q = (int)((word >> (4 * (k & 7))) & 0xFu);
    float prod = (float)(q - 7) * h2f(s_row[k >> 5]); /* exact in fp32 */
    w_row[k] = f2h(prod);                             /* the single fp16 rounding */
  }
}

/* w[N,K] (fp16 bits) = decode(Wq[N,K/8], S[N,K/32]).  Returns 0, or -1 on bad sizes. */
int q4f16_oracle_dequantize(const uint32_t* wq, const uint16_t* s, uint16_t* w, int64_t N, int64_t K,
                            int nthreads) {
  if (N < 0 || K < 0 || (K % 32) != 0) return -1;
#ifdef _OPENMP
  if (nthreads > 0) omp_set_num_threads(nthreads);
#endif
#pragma omp parallel for schedule(static)
  for (int64_t n = 0; n < N; ++n) decode_row(wq + n * (K / 8), s + n * (K / 32), w + n * K, K);
  return 0;
}

/*
 * y[M,N] (fp16 bits) = x[M,K] . decode(Wq,S)^T with fp32 accumulation, k ascending from 0.
 * acc32 (may be NULL) receives the unrounded fp32 sums.
 * Rows of W are independent, so the loop over n is the parallel one; within one (m,n)
 * the sum over k is strictly sequential, as the unscheduled TIR reduction is.
 */
int q4f16_oracle_matmul(const uint16_t* x, const uint32_t* wq, const uint16_t* s, uint16_t* y, float* acc32,
                        int64_t M, int64_t N, int64_t K, int nthreads) {
  if (M < 0 || N < 0 || K < 0 || (K % 32) != 0) return -1;
#ifdef _OPENMP
  if (nthreads > 0) omp_set_num_threads(nthreads);
#endif
  /* x converted once to fp32: f32(x[m,k]) */
  float* xf = (float*)malloc(sizeof(float) * (size_t)(M * K + 1));
  if (!xf) return -2;
  for (int64_t i = 0; i < M * K; ++i) xf[i] = h2f(x[i]);
  int rc = 0;
#pragma omp parallel
  {
    uint16_t* wrow = (uint16_t*)malloc(sizeof(uint16_t) * (size_t)(K + 1));
    float* wf = (float*)malloc(sizeof(float) * (size_t)(K + 1));
    if (!wrow || !wf) {
#pragma omp atomic write
      rc = -2;
    } else {
#pragma omp for schedule(static)
      for (int64_t n = 0; n < N; ++n) {
        decode_row(wq + n * (K / 8), s + n * (K / 32), wrow, K);
        for (int64_t k = 0; k < K; ++k) wf[k] = h2f(wrow[k]);
        for (int64_t m = 0; m < M; ++m) {
          const float* xm = xf + m * K;
          float acc = 0.0f;
          for (int64_t k = 0; k < K; ++k) acc = acc + xm[k] * wf[k];
          if (acc32) acc32[m * N + n] = acc;
          y[m * N + n] = f2h(acc);
        }
      }
    }
    free(wrow);
    free(wf);
  }
  free(xf);
  return rc;
}

/*
 * The unfused form the reference executes when decode and matmul stay two kernels:
 * materialise W fp16 [N,K] in memory, then run the matmul over it.  Same results as
 * q4f16_oracle_matmul; kept so the CPU baseline can be timed in the reference's shape.
 * w_tmp must hold N*K fp16 values.
 */
int q4f16_oracle_matmul_unfused(const uint16_t* x, const uint32_t* wq, const uint16_t* s, uint16_t* w_tmp,
                                uint16_t* y, int64_t M, int64_t N, int64_t K, int nthreads) {
  int rc = q4f16_oracle_dequantize(wq, s, w_tmp, N, K, nthreads);
  if (rc) return rc;
#pragma omp parallel for schedule(static)
  for (int64_t n = 0; n < N; ++n) {
    const uint16_t* wrow = w_tmp + n * K;
    for (int64_t m = 0; m < M; ++m) {
      const uint16_t* xm = x + m * K;
      float acc = 0.0f;
      for (int64_t k = 0; k < K; ++k) acc = acc + h2f(xm[k]) * h2f(wrow[k]);
      y[m * N + n] = f2h(acc);
    }
  }
  return 0;
}

int q4f16_oracle_max_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}
