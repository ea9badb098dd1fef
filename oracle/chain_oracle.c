/* CPU restatement of the reference's fused GEMM-chain arithmetic.
 *
 * TEST INFRASTRUCTURE ONLY: this file is the checker for the CUDA kernels and
 * the timed CPU baseline of the benchmark.  Nothing in the shipped package may
 * call it; the product path has no CPU fallback.
 *
 * Parity status: pinned at the level of the reference's CPU micro-kernels, unpinned above it.
 * The reference's build (TVM + LLVM) is not available, so its generated kernels - the GPU WMMA
 * code in particular - cannot run, and it holds no golden vectors for these chains.  What can run
 * are the two hand-written CPU micro-kernels its Python emits as C++/asm text (6 x 16 AVX2 GEMM
 * tile, AVX-512 exponential; python/ditto/auto_tensorize/intrinsic.py:274-604, 1480-1672):
 * oracle/build_ref.py compiles them as they are, oracle/ref_microkernels.py drives the reference's
 * three CPU chains through them, and tests/golden/ref_microkernels.npz holds those outputs.
 * oracle_exp_ref_literal, oracle_bmm_softmax_bmm_cpu_literal and baseline_chain_fp32 below
 * reproduce them bit for bit; oracle_gemm_act_gemm to 1e-6 (tests/test_oracle.py).  The fp16 /
 * bf16 forms the GPU tests use (rounded intermediates, stable softmax with a scale) share that
 * arithmetic but have no reference output to be compared with: for them parity is unpinned.
 * What the reference's own tests assert is reproduced in tests/ as well: its fp32 build of the
 * attention chain equals torch.bmm -> softmax -> bmm within rtol = atol = 0.1 at
 * (batch, M, N, K, L) = (12, 512, 64, 64, 512), inputs U(-1, 1)
 * (testing/hyper_fusion/bmm_softmax_bmm_wmma_m16n16k16_fp16fp16fp32.py:552-587),
 * and its GEMM micro-kernel equals numpy on all-ones inputs
 * (python_test/auto_tensorize/test_cpu_intrin.py:1013-1096).
 *
 * Shape tuple as in the reference: A [batch, M, K], B [batch, K, L],
 * C [batch, L, N], out [batch, M, N]; all arrays float32, compact row-major.
 * `in_dtype` selects the storage type the reference casts intermediates to:
 * 0 = float16, 1 = bfloat16, 2 = float32 (no rounding).  Inputs are expected to
 * be already representable in that type.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#if defined(__AVX2__) && defined(__FMA__)
#include <immintrin.h>
#endif

#ifdef _OPENMP
#include <omp.h>
#endif

/* ---------------------------------------------------------------- rounding */
static float round_bf16(float x) {
  uint32_t u;
  memcpy(&u, &x, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return x; /* NaN */
  u += 0x7fffu + ((u >> 16) & 1u);               /* round to nearest even */
  u &= 0xffff0000u;
  memcpy(&x, &u, 4);
  return x;
}

/* float -> IEEE half -> float, round to nearest even, overflow to inf. */
static float round_fp16(float x) {
  uint32_t u;
  memcpy(&u, &x, 4);
  const uint32_t sign = u & 0x80000000u;
  uint32_t a = u & 0x7fffffffu;
  float r;
  if (a >= 0x7f800000u) return x;      /* inf / NaN */
  if (a >= 0x477ff000u) {              /* >= 65520 rounds to inf */
    a = 0x7f800000u;
  } else if (a < 0x38800000u) {        /* below 2^-14: half subnormal, spacing 2^-24 */
    float f;
    memcpy(&f, &a, 4);
    f = f * 16777216.0f;               /* exact scaling by 2^24 */
    f = nearbyintf(f);                 /* ties to even in the default rounding mode */
    f = f * (1.0f / 16777216.0f);
    memcpy(&a, &f, 4);
  } else {
    a += 0xfffu + ((a >> 13) & 1u);
    a &= 0xffffe000u;
  }
  a |= sign;
  memcpy(&r, &a, 4);
  return r;
}

static float round_to(float x, int in_dtype) {
  if (in_dtype == 0) return round_fp16(x);
  if (in_dtype == 1) return round_bf16(x);
  return x;
}

/* Exported so the tests can check the rounding helpers against numpy / torch. */
void oracle_round(const float* src, float* dst, long n, int in_dtype) {
  for (long i = 0; i < n; ++i) dst[i] = round_to(src[i], in_dtype);
}

/* ---------------------------------------------------------------- chains */

/* Attention chain exactly as the reference defines it
 * (python/ditto/auto_compute/nn/functional/bmm_chain.py:40-103):
 *   D = A B (fp32 accumulate); P = in_dtype(exp(D)); E = P [C | 1] (fp32 accumulate, the
 *   appended ones column yields the row sum); F = in_dtype(E) / (in_dtype(rowsum) + 1e-5).
 * No scale and no max subtraction: exp overflows once a logit passes ~11 (fp16) / ~88 (fp32).
 * The division and the 1e-5 are carried out in in_dtype like the generated code does. */
void oracle_bmm_softmax_bmm_literal(const float* A, const float* B, const float* C, float* F, int batch, int M,
                                    int N, int K, int L, int in_dtype) {
#pragma omp parallel
  {
    float* p = (float*)malloc(sizeof(float) * (size_t)L);
    float* e = (float*)malloc(sizeof(float) * (size_t)N);
#pragma omp for collapse(2) schedule(static)
    for (int b = 0; b < batch; ++b) {
      for (int m = 0; m < M; ++m) {
        const float* a = A + ((size_t)b * M + m) * K;
        const float* Bb = B + (size_t)b * K * L;
        const float* Cb = C + (size_t)b * L * N;
        for (int l = 0; l < L; ++l) p[l] = 0.f;
        for (int k = 0; k < K; ++k) {
          const float av = a[k];
          const float* brow = Bb + (size_t)k * L;
          for (int l = 0; l < L; ++l) p[l] += av * brow[l];
        }
        float sum = 0.f;
        for (int n = 0; n < N; ++n) e[n] = 0.f;
        for (int l = 0; l < L; ++l) {
          const float pv = round_to(expf(p[l]), in_dtype);
          sum += pv;
          const float* crow = Cb + (size_t)l * N;
          for (int n = 0; n < N; ++n) e[n] += pv * crow[n];
        }
        const float den = round_to(round_to(sum, in_dtype) + round_to(1e-5f, in_dtype), in_dtype);
        float* f = F + ((size_t)b * M + m) * N;
        for (int n = 0; n < N; ++n) f[n] = round_to(round_to(e[n], in_dtype) / den, in_dtype);
      }
    }
    free(p);
    free(e);
  }
}

/* ------------------------------------------------------------------------------------------
 * The reference's CPU exponential, step by step as its AVX-512 micro-kernel performs it
 * (python/ditto/auto_tensorize/intrinsic.py:1480-1672): clamp to +-88.376, n = floor(x log2(e) + 0.5),
 * r = (n C2) - ((n C1) - x), y = ((((((p0 r + p1) r + p2) r + p3) r + p4) r + p5) r) r + r + 1,
 * result y * 2^n; every product and sum rounded separately (no fused multiply-add).  Note the
 * sign of the C2 term: the Cephes reduction is x - n C1 - n C2, the kernel computes
 * x - n C1 + n C2, so its result is exp(x) * exp(2 n C2) ~ exp(x) (1 - 4.24e-4 n).  The
 * restatement keeps that, bit for bit, because the reference's CPU results contain it. */
#if defined(__GNUC__) && !defined(__clang__)
__attribute__((optimize("fp-contract=off")))
#endif
void oracle_exp_ref_literal(const float* x, float* y, long n) {
  const float hi = 88.3762626647949f, lo = -88.3762626647949f, log2e = 1.44269504088896341f;
  const float c1 = 0.693359375f, c2 = -2.12194440e-4f;
  const float p0 = 1.9875691500E-4f, p1 = 1.3981999507E-3f, p2 = 8.3334519073E-3f, p3 = 4.1665795894E-2f,
              p4 = 1.6666665459E-1f, p5 = 5.0000001201E-1f;
  for (long i = 0; i < n; ++i) {
    volatile float v = x[i];
    v = v < hi ? v : hi;
    v = v > lo ? v : lo;
    volatile float fx = v * log2e;
    fx = fx + 0.5f;
    volatile float t = (float)(int32_t)fx;        /* truncation, then back to float */
    if (t > fx) t = t - 1.0f;                      /* -> floor */
    volatile float a = t * c1;
    a = a - v;
    volatile float r = t * c2;
    r = r - a;
    volatile float q = p0 * r;
    q = q + p1; q = q * r;
    q = q + p2; q = q * r;
    q = q + p3; q = q * r;
    q = q + p4; q = q * r;
    q = q + p5; q = q * r;
    q = q * r;
    q = q + r;
    q = q + 1.0f;
    union { int32_t i; float f; } pw;
    pw.i = (int32_t)(((uint32_t)((int32_t)t + 0x7f)) << 23);
    y[i] = q * pw.f;
  }
}

/* The reference's CPU attention chain (benchmark/chimera/cpu/bmm_softmax_bmm.py:64-170): fp32,
 * exp without max subtraction (the exponential above), the row sum obtained from a column of ones
 * appended to V at index N, one division, no epsilon.  Both products accumulate along the reduction
 * index in order with fused multiply-adds, which is what the 6 x 16 micro-kernel does for each
 * output element (intrinsic.py:274-604), so the result equals the micro-kernel-driven evaluation
 * bit for bit. */
void oracle_bmm_softmax_bmm_cpu_literal(const float* A, const float* B, const float* C, float* F, int batch, int M,
                                        int N, int K, int L) {
#pragma omp parallel
  {
    float* d = (float*)malloc(sizeof(float) * (size_t)L);
    float* p = (float*)malloc(sizeof(float) * (size_t)L);
#pragma omp for collapse(2) schedule(static)
    for (int b = 0; b < batch; ++b) {
      for (int m = 0; m < M; ++m) {
        const float* a = A + ((size_t)b * M + m) * K;
        const float* Bb = B + (size_t)b * K * L;
        const float* Cb = C + (size_t)b * L * N;
        for (int l = 0; l < L; ++l) {
          float acc = 0.f;
          for (int k = 0; k < K; ++k) acc = fmaf(a[k], Bb[(size_t)k * L + l], acc);
          d[l] = acc;
        }
        oracle_exp_ref_literal(d, p, L);
        float sum = 0.f;
        for (int l = 0; l < L; ++l) sum = fmaf(p[l], 1.0f, sum);
        float* f = F + ((size_t)b * M + m) * N;
        for (int n = 0; n < N; ++n) {
          float acc = 0.f;
          for (int l = 0; l < L; ++l) acc = fmaf(p[l], Cb[(size_t)l * N + n], acc);
          f[n] = acc / sum;
        }
      }
    }
    free(d);
    free(p);
  }
}

/* The same function in max-subtracted form with an explicit scale:
 *   F = softmax(scale * A B) C, P rounded to in_dtype before the second product
 *   (mirrors the reference's cast of the intermediate, bmm_chain.py:64-70), output left in fp32.
 * For scale = 1 and logits small enough not to overflow it equals the literal form up to the
 * 1e-5 term and rounding.  `wide` != 0 accumulates in double (cross-check of the fp32 path). */
void oracle_bmm_softmax_bmm(const float* A, const float* B, const float* C, float* F, int batch, int M, int N, int K,
                            int L, float scale, int in_dtype, int wide) {
#pragma omp parallel
  {
    double* s = (double*)malloc(sizeof(double) * (size_t)L);
    double* e = (double*)malloc(sizeof(double) * (size_t)N);
    float* sf = (float*)malloc(sizeof(float) * (size_t)L);
#pragma omp for collapse(2) schedule(static)
    for (int b = 0; b < batch; ++b) {
      for (int m = 0; m < M; ++m) {
        const float* a = A + ((size_t)b * M + m) * K;
        const float* Bb = B + (size_t)b * K * L;
        const float* Cb = C + (size_t)b * L * N;
        if (wide) {
          for (int l = 0; l < L; ++l) s[l] = 0.0;
          for (int k = 0; k < K; ++k) {
            const double av = a[k];
            const float* brow = Bb + (size_t)k * L;
            for (int l = 0; l < L; ++l) s[l] += av * (double)brow[l];
          }
        } else {
          for (int l = 0; l < L; ++l) sf[l] = 0.f;
          for (int k = 0; k < K; ++k) {
            const float av = a[k];
            const float* brow = Bb + (size_t)k * L;
            for (int l = 0; l < L; ++l) sf[l] += av * brow[l];
          }
          for (int l = 0; l < L; ++l) s[l] = (double)sf[l];
        }
        double mx = -INFINITY;
        for (int l = 0; l < L; ++l) mx = s[l] > mx ? s[l] : mx;
        double sum = 0.0;
        for (int n = 0; n < N; ++n) e[n] = 0.0;
        for (int l = 0; l < L; ++l) {
          double pv = wide ? exp((s[l] - mx) * (double)scale) : (double)expf((float)((s[l] - mx) * (double)scale));
          sum += pv;
          pv = (double)round_to((float)pv, in_dtype);
          const float* crow = Cb + (size_t)l * N;
          if (wide) {
            for (int n = 0; n < N; ++n) e[n] += pv * (double)crow[n];
          } else {
            for (int n = 0; n < N; ++n) e[n] = (double)((float)e[n] + (float)pv * crow[n]);
          }
        }
        float* f = F + ((size_t)b * M + m) * N;
        for (int n = 0; n < N; ++n) f[n] = (float)(e[n] / sum);
      }
    }
    free(s);
    free(e);
    free(sf);
  }
}

/* GEMM chain F = act(A B) C with the intermediate cast to in_dtype, fp32 accumulate:
 *   act = 0: identity -- BatchGemmGemm (benchmark/chimera/cpu/bmm_bmm_cpu.py:55-116,
 *            GPU twin benchmark/chimera/cuda/bmm_bmm_cuda.py:69-150)
 *   act = 1: ReLU as if_then_else(D > 0, D, 0) -- BatchGemmReluGemm
 *            (python_test/auto_tensorize/test_hyper_fusion_cpu.py:24-96).
 * Output left in fp32 (round it with oracle_round for the 16-bit outputs). */
void oracle_gemm_act_gemm(const float* A, const float* B, const float* C, float* F, int batch, int M, int N, int K,
                          int L, int act, int in_dtype, int wide) {
#pragma omp parallel
  {
    double* h = (double*)malloc(sizeof(double) * (size_t)L);
    double* e = (double*)malloc(sizeof(double) * (size_t)N);
    float* hf = (float*)malloc(sizeof(float) * (size_t)L);
    float* ef = (float*)malloc(sizeof(float) * (size_t)N);
#pragma omp for collapse(2) schedule(static)
    for (int b = 0; b < batch; ++b) {
      for (int m = 0; m < M; ++m) {
        const float* a = A + ((size_t)b * M + m) * K;
        const float* Bb = B + (size_t)b * K * L;
        const float* Cb = C + (size_t)b * L * N;
        float* f = F + ((size_t)b * M + m) * N;
        if (wide) {
          for (int l = 0; l < L; ++l) h[l] = 0.0;
          for (int k = 0; k < K; ++k) {
            const double av = a[k];
            const float* brow = Bb + (size_t)k * L;
            for (int l = 0; l < L; ++l) h[l] += av * (double)brow[l];
          }
          for (int n = 0; n < N; ++n) e[n] = 0.0;
          for (int l = 0; l < L; ++l) {
            float hv = (float)h[l];
            if (act == 1) hv = hv > 0.f ? hv : 0.f;
            const double hr = (double)round_to(hv, in_dtype);
            const float* crow = Cb + (size_t)l * N;
            for (int n = 0; n < N; ++n) e[n] += hr * (double)crow[n];
          }
          for (int n = 0; n < N; ++n) f[n] = (float)e[n];
        } else {
          for (int l = 0; l < L; ++l) hf[l] = 0.f;
          for (int k = 0; k < K; ++k) {
            const float av = a[k];
            const float* brow = Bb + (size_t)k * L;
            for (int l = 0; l < L; ++l) hf[l] += av * brow[l];
          }
          for (int n = 0; n < N; ++n) ef[n] = 0.f;
          for (int l = 0; l < L; ++l) {
            float hv = hf[l];
            if (act == 1) hv = hv > 0.f ? hv : 0.f;
            hv = round_to(hv, in_dtype);
            const float* crow = Cb + (size_t)l * N;
            for (int n = 0; n < N; ++n) ef[n] += hv * crow[n];
          }
          for (int n = 0; n < N; ++n) f[n] = ef[n];
        }
      }
    }
    free(h);
    free(e);
    free(hf);
    free(ef);
  }
}

/* ---------------------------------------------------------------- timed CPU baseline
 * Port of the loop structure the reference's CPU scheduler produces
 * (src/auto_tensorize/hyper_fusion_cpu.cc:644-907: a parallel outer loop over batch x row
 * blocks, the first GEMM's tile for one row block computed into a cache-resident buffer, the
 * element-wise stage applied there, then the second GEMM consuming it) around a 6 x 16 fp32
 * FMA register tile like the AVX2 micro-kernel the reference generates
 * (python/ditto/auto_tensorize/intrinsic.py:274-604).  fp32 throughout, like the reference's
 * CPU runs.  kind: 0 = softmax (stable form, `scale`), 1 = ReLU, 2 = identity. */

#define MR 6
#define NR 16

#if defined(__AVX2__) && defined(__FMA__)
/* acc[MR][NR] += A[MR x kc] (row stride lda) * B[kc x NR] (row stride ldb) */
static void micro_6x16(const float* A, int lda, const float* B, int ldb, float* Cc, int ldc, int kc, int rows) {
  __m256 c[MR][2];
  for (int i = 0; i < MR; ++i) {
    c[i][0] = _mm256_setzero_ps();
    c[i][1] = _mm256_setzero_ps();
  }
  for (int k = 0; k < kc; ++k) {
    const __m256 b0 = _mm256_loadu_ps(B + (size_t)k * ldb);
    const __m256 b1 = _mm256_loadu_ps(B + (size_t)k * ldb + 8);
    for (int i = 0; i < MR; ++i) {
      const __m256 a = _mm256_broadcast_ss(A + (size_t)(i < rows ? i : 0) * lda + k);
      c[i][0] = _mm256_fmadd_ps(a, b0, c[i][0]);
      c[i][1] = _mm256_fmadd_ps(a, b1, c[i][1]);
    }
  }
  for (int i = 0; i < rows; ++i) {
    float* dst = Cc + (size_t)i * ldc;
    _mm256_storeu_ps(dst, _mm256_add_ps(_mm256_loadu_ps(dst), c[i][0]));
    _mm256_storeu_ps(dst + 8, _mm256_add_ps(_mm256_loadu_ps(dst + 8), c[i][1]));
  }
}
#else
static void micro_6x16(const float* A, int lda, const float* B, int ldb, float* Cc, int ldc, int kc, int rows) {
  for (int i = 0; i < rows; ++i)
    for (int k = 0; k < kc; ++k)
      for (int j = 0; j < NR; ++j) Cc[(size_t)i * ldc + j] += A[(size_t)i * lda + k] * B[(size_t)k * ldb + j];
}
#endif

/* Requires L % 16 == 0 and N % 16 == 0 (the reference asserts the same on its tiles). */
int baseline_chain_fp32(const float* A, const float* B, const float* C, float* F, int batch, int M, int N, int K,
                        int L, int kind, float scale, int threads) {
  if (L % NR || N % NR) return -1;
  const int row_blocks = (M + MR - 1) / MR;
#ifdef _OPENMP
  if (threads > 0) omp_set_num_threads(threads);
#else
  (void)threads;
#endif
#pragma omp parallel
  {
    float* d = (float*)aligned_alloc(64, sizeof(float) * (size_t)MR * L);
#pragma omp for collapse(2) schedule(static)
    for (int b = 0; b < batch; ++b) {
      for (int rb = 0; rb < row_blocks; ++rb) {
        const int m0 = rb * MR;
        const int rows = M - m0 < MR ? M - m0 : MR;
        const float* a = A + ((size_t)b * M + m0) * K;
        const float* Bb = B + (size_t)b * K * L;
        const float* Cb = C + (size_t)b * L * N;
        float* f = F + ((size_t)b * M + m0) * N;
        memset(d, 0, sizeof(float) * (size_t)MR * L);
        for (int l0 = 0; l0 < L; l0 += NR) micro_6x16(a, K, Bb + l0, L, d + l0, L, K, rows);
        float inv[MR];
        for (int i = 0; i < rows; ++i) {
          float* row = d + (size_t)i * L;
          inv[i] = 1.f;
          if (kind == 0) {
            float mx = row[0];
            for (int l = 1; l < L; ++l) mx = row[l] > mx ? row[l] : mx;
            float sum = 0.f;
            for (int l = 0; l < L; ++l) {
              row[l] = expf((row[l] - mx) * scale);
              sum += row[l];
            }
            inv[i] = 1.f / sum;
          } else if (kind == 1) {
            for (int l = 0; l < L; ++l) row[l] = row[l] > 0.f ? row[l] : 0.f;
          }
        }
        for (int i = 0; i < rows; ++i) memset(f + (size_t)i * N, 0, sizeof(float) * (size_t)N);
        for (int n0 = 0; n0 < N; n0 += NR) micro_6x16(d, L, Cb + n0, N, f + n0, N, L, rows);
        if (kind == 0)
          for (int i = 0; i < rows; ++i)
            for (int n = 0; n < N; ++n) f[(size_t)i * N + n] *= inv[i];
      }
    }
    free(d);
  }
  return 0;
}

int oracle_max_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/* Position-wise feed-forward block  F = act2(in_dtype(act1(A B + b1)) C + b2), fp32 accumulate
 * (wide: fp64): PositionwiseFeedForward, python/ditto/auto_compute/nn/model/transformer.py:21-34, with
 * linear + bias as in nn/functional/linear.py:4-41.  act: 0 identity, 1 ReLU (activation.py:9-26),
 * 2 GELU in the reference's tanh form (activation.py:29-39).  b1 [batch, L], b2 [batch, N] or NULL. */
static double act_d(double v, int act) {
  if (act == 1) return v > 0.0 ? v : 0.0;
  if (act == 2) return 0.5 * v * (1.0 + tanh(v * 0.7978845608 * (1.0 + 0.044715 * v * v)));
  return v;
}

void oracle_ffn(const float* A, const float* B, const float* b1, const float* C, const float* b2, float* F, int batch,
                int M, int N, int K, int L, int act1, int act2, int in_dtype) {
#pragma omp parallel
  {
    double* h = (double*)malloc(sizeof(double) * (size_t)L);
    double* e = (double*)malloc(sizeof(double) * (size_t)N);
#pragma omp for collapse(2) schedule(static)
    for (int b = 0; b < batch; ++b) {
      for (int m = 0; m < M; ++m) {
        const float* a = A + ((size_t)b * M + m) * K;
        const float* Bb = B + (size_t)b * K * L;
        const float* Cb = C + (size_t)b * L * N;
        float* f = F + ((size_t)b * M + m) * N;
        for (int l = 0; l < L; ++l) h[l] = 0.0;
        for (int k = 0; k < K; ++k) {
          const double av = a[k];
          const float* brow = Bb + (size_t)k * L;
          for (int l = 0; l < L; ++l) h[l] += av * (double)brow[l];
        }
        for (int n = 0; n < N; ++n) e[n] = 0.0;
        for (int l = 0; l < L; ++l) {
          double hv = (double)(float)h[l] + (b1 ? (double)b1[(size_t)b * L + l] : 0.0);
          const double hr = (double)round_to((float)act_d(hv, act1), in_dtype);
          const float* crow = Cb + (size_t)l * N;
          for (int n = 0; n < N; ++n) e[n] += hr * (double)crow[n];
        }
        for (int n = 0; n < N; ++n) f[n] = (float)act_d((double)(float)e[n] + (b2 ? (double)b2[(size_t)b * N + n] : 0.0), act2);
      }
    }
    free(h);
    free(e);
  }
}
