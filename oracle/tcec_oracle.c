/*
 * CPU restatement of wmma_extension's TCEC arithmetic.  TEST INFRASTRUCTURE ONLY:
 * it is the checker that tests, the smoke test and the bench's CPU-baseline leg
 * compare the CUDA library against; nothing in the library calls it.
 *
 * Parity status: the split (hi / scaled lo) is pinned bit for bit against the
 * reference's own device code run on a B200 (fixtures under tests/golden/,
 * produced by tests/golden/make_golden.py from oracle/_ref).  The products are
 * pinned to a tolerance only: the reference runs them on tensor cores whose
 * internal rounding is not specified, so this file models a tensor-core product
 * as an exact dot product of the block rounded once to FP32.
 *
 * The reference has no CPU implementation of the path (its scale helpers are
 * __device__ only and its host to_tf32 returns the input unrounded,
 * include/wmma_extension/detail/common.hpp:46-48), so roundings are done here
 * in integer arithmetic.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

static uint32_t f2u(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  return u;
}
static float u2f(uint32_t u) {
  float f;
  memcpy(&f, &u, 4);
  return f;
}

/* FP32 -> FP16 -> FP32, round to nearest even: static_cast<half>(float),
 * include/wmma_extension/detail/common.hpp:25-28. */
float oracle_round_fp16(float v) {
  const uint32_t x = f2u(v);
  const uint32_t sign = x & 0x80000000u;
  const int exp = (int)((x >> 23) & 0xff);
  uint32_t man = x & 0x7fffffu;
  if (exp == 0xff) return v; /* inf / nan */
  const int e = exp - 127 + 15;
  uint32_t h; /* fp16 magnitude bits */
  if (e >= 31) {
    h = 0x7c00u;
  } else if (e <= 0) {
    const int shift = 14 - e; /* >= 14 */
    if (exp == 0 || shift > 24) {
      h = 0u; /* below half of the smallest fp16 subnormal */
    } else {
      man |= 0x800000u;
      const uint32_t q = man >> shift;
      const uint32_t rem = man & ((1u << shift) - 1u);
      const uint32_t half = 1u << (shift - 1);
      h = q;
      if (rem > half || (rem == half && (q & 1u))) h += 1u;
    }
  } else {
    h = ((uint32_t)e << 10) | (man >> 13);
    const uint32_t rem = man & 0x1fffu;
    if (rem > 0x1000u || (rem == 0x1000u && (h & 1u))) h += 1u; /* may carry up to inf */
  }
  /* widen back */
  const uint32_t he = (h >> 10) & 0x1f, hm = h & 0x3ffu;
  float r;
  if (he == 0x1f) {
    r = u2f(0x7f800000u);
  } else if (he == 0) {
    r = (float)hm * 5.9604644775390625e-08f; /* 2^-24 */
  } else {
    r = u2f(((he - 15 + 127) << 23) | (hm << 13));
  }
  return sign ? -r : r;
}

/* cvt.rna.tf32.f32: nearest, ties away from zero, low 13 bits cleared
 * (include/wmma_extension/detail/common.hpp:37-45). */
float oracle_round_tf32(float v) {
  const uint32_t x = f2u(v);
  if (((x >> 23) & 0xff) == 0xff) return v;
  return u2f((x + 0x1000u) & 0xffffe000u);
}

/* policy: 0 = fp16, 1 = tf32 (input type only). */
static float round_t(float v, int tf32) { return tf32 ? oracle_round_tf32(v) : oracle_round_fp16(v); }

/* hv = cast<T>(v); dhv = cast<T>(scale0<T>(v - float(hv)))
 * include/wmma_extension/tcec/tcec.hpp:219-223, scale.hpp:8-13. */
void oracle_split(const float* in, float* hi, float* lo, size_t n, int tf32) {
  const float s = tf32 ? 1.0f : 2048.0f;
  for (size_t i = 0; i < n; ++i) {
    const float h = round_t(in[i], tf32);
    hi[i] = h;
    if (lo) lo[i] = round_t((in[i] - h) * s, tf32);
  }
}

static float to_f32_rz(double d) {
  float f = (float)d;
  if (fabs((double)f) > fabs(d)) f = nextafterf(f, 0.0f);
  return f;
}

static double at(const float* p, int col_major, long long ld, int i, int j) {
  return col_major ? p[(long long)j * ld + i] : p[(long long)i * ld + j];
}

/*
 * C = alpha * A*B + beta * C following the reference's arithmetic:
 *   per block of `fk` along K (16 for fp16, 8 for tf32; policy.hpp:68-99)
 *     tmp  = TC(A_hi, B_hi, 0)            tcec.hpp:673-675, 689-691
 *     main = main + tmp  (FP32 RN add)    tcec.hpp:676-679, 692-694
 *     corr = TC(A_lo, B_hi, corr); corr = TC(A_hi, B_lo, corr)   :680-687, 695-702
 *   out = main + corr / 2048 (fp16) or main + corr (tf32)        :332-336
 *   C   = alpha * out + beta * C          test/tcec/batch_gemm.cu:119-185
 * rn_block: number of fk blocks accumulated by the tensor-core model before
 *   the RN add (1 = reference mma_rn_sync; 0 = whole K, reference mma_rz_sync).
 * tc_rz: the tensor-core model rounds toward zero instead of to nearest.
 * ec == 0: single product, no lo terms (no_cor.hpp:658-701 / 750-804).
 */
void oracle_tcec_gemm(int a_col, int b_col, int c_col, int m, int n, int k, float alpha,
                      const float* a, long long lda, const float* b, long long ldb, float beta,
                      float* c, long long ldc, int tf32, int ec, int rn_block, int tc_rz) {
  const int fk = tf32 ? 8 : 16;
  const float s1 = tf32 ? 1.0f : (1.0f / 2048.0f);
  float *ah = 0, *al = 0, *bh = 0, *bl = 0;
  /* split once into K-contiguous scratch */
  ah = (float*)__builtin_malloc(sizeof(float) * (size_t)m * k * 2);
  bh = (float*)__builtin_malloc(sizeof(float) * (size_t)n * k * 2);
  al = ah + (size_t)m * k;
  bl = bh + (size_t)n * k;
  for (int i = 0; i < m; ++i)
    for (int l = 0; l < k; ++l) {
      const float v = (float)at(a, a_col, lda, i, l);
      const float h = round_t(v, tf32);
      ah[(size_t)i * k + l] = h;
      al[(size_t)i * k + l] = round_t((v - h) * (tf32 ? 1.0f : 2048.0f), tf32);
    }
  for (int j = 0; j < n; ++j)
    for (int l = 0; l < k; ++l) {
      const float v = (float)at(b, b_col, ldb, l, j);
      const float h = round_t(v, tf32);
      bh[(size_t)j * k + l] = h;
      bl[(size_t)j * k + l] = round_t((v - h) * (tf32 ? 1.0f : 2048.0f), tf32);
    }
  const int chunk = rn_block > 0 ? rn_block * fk : (k > 0 ? k : 1);
#pragma omp parallel for collapse(2) schedule(static)
  for (int i = 0; i < m; ++i)
    for (int j = 0; j < n; ++j) {
      const float* pah = ah + (size_t)i * k;
      const float* pal = al + (size_t)i * k;
      const float* pbh = bh + (size_t)j * k;
      const float* pbl = bl + (size_t)j * k;
      float main_acc = 0.f, corr = 0.f;
      for (int k0 = 0; k0 < k; k0 += chunk) {
        const int k1 = k0 + chunk < k ? k0 + chunk : k;
        float tmp = 0.f;
        for (int kk = k0; kk < k1; kk += fk) {
          const int ke = kk + fk < k1 ? kk + fk : k1;
          double d = 0.0, dc1 = 0.0, dc2 = 0.0;
          for (int l = kk; l < ke; ++l) {
            d += (double)pah[l] * (double)pbh[l];
            dc1 += (double)pal[l] * (double)pbh[l];
            dc2 += (double)pah[l] * (double)pbl[l];
          }
          tmp = tc_rz ? to_f32_rz((double)tmp + d) : (float)((double)tmp + d);
          if (ec) {
            corr = tc_rz ? to_f32_rz((double)corr + dc1) : (float)((double)corr + dc1);
            corr = tc_rz ? to_f32_rz((double)corr + dc2) : (float)((double)corr + dc2);
          }
        }
        main_acc = main_acc + tmp;
      }
      float out = ec ? main_acc + corr * s1 : main_acc;
      float* pc = c_col ? &c[(long long)j * ldc + i] : &c[(long long)i * ldc + j];
      out = alpha * out;
      if (beta != 0.f) out += beta * *pc;
      *pc = out;
    }
  __builtin_free(ah);
  __builtin_free(bh);
}

/* FP64 host GEMM, the reference's ground truth: test/tcec/batch_gemm.cu:561-575
 * (OpenMP) and test/tcec/mma.cu:130-154.  Rows [row0, row1) only, so a bounded
 * sample of a large problem can be checked or timed. */
void oracle_gemm_f64(int a_col, int b_col, int m, int n, int k, const float* a, long long lda,
                     const float* b, long long ldb, double* c, long long ldc, int row0, int row1) {
  (void)m;
  if (!b_col && !a_col) {
    /* both row-major: walk B along its rows so the host caches see unit stride */
#pragma omp parallel for schedule(static)
    for (int i = row0; i < row1; ++i) {
      double* ci = c + (long long)(i - row0) * ldc;
      for (int j = 0; j < n; ++j) ci[j] = 0.0;
      for (int l = 0; l < k; ++l) {
        const double av = (double)a[(long long)i * lda + l];
        const float* bl = b + (long long)l * ldb;
        for (int j = 0; j < n; ++j) ci[j] += av * (double)bl[j];
      }
    }
    return;
  }
#pragma omp parallel for collapse(2) schedule(static)
  for (int i = row0; i < row1; ++i)
    for (int j = 0; j < n; ++j) {
      double s = 0.0;
      for (int l = 0; l < k; ++l) s += at(a, a_col, lda, i, l) * at(b, b_col, ldb, l, j);
      c[(long long)(i - row0) * ldc + j] = s;
    }
}

/* FP32 sequential-FMA GEMM: the accuracy class of an FP32 SIMT SGEMM (the
 * reference's op_simt policy, tcec/detail/simt/detail/m16n16k16.hpp:303-355,
 * accumulates with FP32 FMAs). */
void oracle_gemm_f32(int a_col, int b_col, int m, int n, int k, const float* a, long long lda,
                     const float* b, long long ldb, float* c, long long ldc, int row0, int row1) {
  (void)m;
#pragma omp parallel for collapse(2) schedule(static)
  for (int i = row0; i < row1; ++i)
    for (int j = 0; j < n; ++j) {
      float s = 0.f;
      for (int l = 0; l < k; ++l)
        s = fmaf((float)at(a, a_col, lda, i, l), (float)at(b, b_col, ldb, l, j), s);
      c[(long long)(i - row0) * ldc + j] = s;
    }
}

/* Error metrics of the reference's tests, against an FP64 result (both row-major, ld = n):
 *   out[0] max|c-r| / max|r|       test/primitive/common.hpp:100-102
 *   out[1] sqrt(sum (c-r)^2 / sum r^2)   test/tcec/batch_gemm.cu:546-575,605
 *   out[2] max|c-r|                test/tcec/mma.cu:152 */
void oracle_errors(const float* c, const double* ref, size_t count, double* out) {
  double maxd = 0, maxr = 0, sd = 0, sr = 0;
  for (size_t i = 0; i < count; ++i) {
    const double d = fabs((double)c[i] - ref[i]);
    if (d > maxd) maxd = d;
    if (fabs(ref[i]) > maxr) maxr = fabs(ref[i]);
    sd += d * d;
    sr += ref[i] * ref[i];
  }
  out[0] = maxr > 0 ? maxd / maxr : maxd;
  out[1] = sr > 0 ? sqrt(sd / sr) : sqrt(sd);
  out[2] = maxd;
}

/* Thread count of the host loops, set explicitly so that a launcher's OMP_NUM_THREADS does not decide it. */
void oracle_set_num_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

int oracle_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}
