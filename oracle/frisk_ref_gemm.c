/*
 * frisk_ref_gemm.c -- CPU oracle for `frisk.gemm`.  TEST INFRASTRUCTURE, NOT PRODUCT CODE:
 * only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline legs may build, load or
 * call it; nothing under frisk_b200/ does.
 *
 * PARITY UNPINNED (numerics): the reference (Xiebaokang/frisk) contains no GEMM arithmetic at
 * all -- no lowering, no kernel, no host loop, and none of its tests runs a GEMM -- so there is
 * no golden vector or reference output to pin these sums against.  What IS taken from the
 * reference is the op's meaning:
 *   - operands and attributes of frisk.gemm: include/Dialect/Frisk/IR/FriskOps.td:248-289
 *     (A, B, C memrefs; transA, transB, M, N, K, clear_accum; C is updated in place);
 *   - shapes: A is [M,K], B is [K,N], C is [M,N] whatever the trans flags are
 *     (ffi/ir.cpp:339-359, lib/Dialect/Frisk/IR/FriskOps.cpp:1264-1283);
 *   - the trans flags give the memory order: K is the inner dimension of A iff !transA and of
 *     B iff transB (lib/Dialect/Frisk/IR/FriskOps.cpp:1359-1360, 1376-1377);
 *   - the dtype vocabulary fp32 / fp16 / bf16 / e4m3fn (ffi/ir.cpp:163-175, 240-245, 410-423).
 * The restatement:  C[m,n] = (clear_accum ? 0 : C[m,n]) + sa[m] * sb[n] * sum_k A[m,k] * B[k,n],
 * inputs decoded exactly to fp32, every product rounded to fp32, summed in fp32 in increasing k
 * (or in fp64 when acc64 is set, for error analysis), one round-to-nearest-even cast to C's type.
 * The storage codecs (fp16, bf16, e4m3fn) are pinned in tests against numpy / ml_dtypes / torch.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

enum { REF_F32 = 0, REF_F16 = 1, REF_BF16 = 2, REF_E4M3 = 3, REF_E5M2 = 4 };

typedef struct frisk_ref_desc {
  int64_t M, N, K;
  int32_t ab_type, c_type;
  int64_t lda, ldb, ldc; /* elements */
  int32_t transA, transB, clear_accum;
  int32_t use_scales; /* sa[M], sb[N] */
  int32_t acc64;      /* accumulate in double instead of float */
} frisk_ref_desc;

static float u32_as_f32(uint32_t u) {
  float f;
  memcpy(&f, &u, 4);
  return f;
}
static uint32_t f32_as_u32(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  return u;
}

float frisk_ref_decode_f16(uint16_t h) {
  const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  const uint32_t exp = (h >> 10) & 0x1Fu;
  const uint32_t man = h & 0x3FFu;
  if (exp == 0) {
    if (man == 0) return u32_as_f32(sign);
    return (sign ? -1.0f : 1.0f) * ldexpf((float)man, -24); /* subnormal */
  }
  if (exp == 31) return u32_as_f32(sign | 0x7F800000u | (man << 13));
  return u32_as_f32(sign | ((exp + 112u) << 23) | (man << 13));
}

float frisk_ref_decode_bf16(uint16_t b) { return u32_as_f32((uint32_t)b << 16); }

/* e4m3fn: 1 sign, 4 exponent (bias 7), 3 mantissa; no infinity; S.1111.111 is NaN; max 448. */
float frisk_ref_decode_e4m3(uint8_t v) {
  const int sign = v >> 7;
  const int exp = (v >> 3) & 0xF;
  const int man = v & 7;
  float r;
  if (exp == 15 && man == 7) return NAN;
  if (exp == 0) r = ldexpf((float)man, -9); /* man/8 * 2^-6 */
  else r = ldexpf(1.0f + (float)man / 8.0f, exp - 7);
  return sign ? -r : r;
}

/* e5m2: 1 sign, 5 exponent (bias 15), 2 mantissa -- the top byte of an IEEE half, infinities and
 * NaNs included. */
float frisk_ref_decode_e5m2(uint8_t v) { return frisk_ref_decode_f16((uint16_t)((uint16_t)v << 8)); }

uint16_t frisk_ref_encode_bf16(float f) {
  uint32_t u = f32_as_u32(f);
  if ((u & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)((u >> 16) | 0x40u); /* quiet NaN */
  u += 0x7FFFu + ((u >> 16) & 1u);                                            /* RNE */
  return (uint16_t)(u >> 16);
}

uint16_t frisk_ref_encode_f16(float f) {
  const uint32_t u = f32_as_u32(f);
  const uint16_t sign = (uint16_t)((u >> 16) & 0x8000u);
  const uint32_t a = u & 0x7FFFFFFFu;
  if (a > 0x7F800000u) return (uint16_t)(sign | 0x7E00u);  /* NaN */
  if (a >= 0x477FF000u) return (uint16_t)(sign | 0x7C00u); /* rounds to >= 65520 -> inf */
  if (a < 0x33000001u) return sign;                        /* <= 2^-25 rounds to zero */
  int32_t e = (int32_t)(a >> 23) - 127;
  uint32_t m = (a & 0x7FFFFFu) | 0x800000u;
  int shift;
  uint32_t base;
  if (e < -14) { /* subnormal half: value = m * 2^(e-23), unit 2^-24 */
    shift = -e - 1; /* 13 + (-14 - e) */
    base = 0;
  } else {
    shift = 13;
    base = (uint32_t)(e + 15) << 10;
    m &= 0x7FFFFFu;
  }
  uint32_t q = m >> shift;
  const uint32_t rem = m & ((1u << shift) - 1u);
  const uint32_t half = 1u << (shift - 1);
  if (rem > half || (rem == half && (q & 1u))) q++;
  return (uint16_t)(sign | (base + q)); /* a mantissa carry moves into the exponent */
}

static float decode_in(const void* p, int64_t i, int type) {
  switch (type) {
    case REF_F32: return ((const float*)p)[i];
    case REF_F16: return frisk_ref_decode_f16(((const uint16_t*)p)[i]);
    case REF_BF16: return frisk_ref_decode_bf16(((const uint16_t*)p)[i]);
    case REF_E4M3: return frisk_ref_decode_e4m3(((const uint8_t*)p)[i]);
    default: return frisk_ref_decode_e5m2(((const uint8_t*)p)[i]);
  }
}

static void store_out(void* p, int64_t i, int type, float v) {
  switch (type) {
    case REF_F32: ((float*)p)[i] = v; break;
    case REF_F16: ((uint16_t*)p)[i] = frisk_ref_encode_f16(v); break;
    default: ((uint16_t*)p)[i] = frisk_ref_encode_bf16(v); break;
  }
}

static int valid_desc(const frisk_ref_desc* d) {
  if (!d || d->M <= 0 || d->N <= 0 || d->K <= 0) return 0;
  if (d->ab_type < 0 || d->ab_type > 4 || d->c_type < 0 || d->c_type > 2) return 0;
  if (d->lda < (d->transA ? d->M : d->K)) return 0;
  if (d->ldb < (d->transB ? d->K : d->N)) return 0;
  if (d->ldc < d->N) return 0;
  return 1;
}

/*
 * Computes rows [m_begin, m_end) of C (all N columns).  Returns 0, or -1 on a bad argument.
 * num_threads <= 0 uses the OpenMP default.
 */
int frisk_ref_gemm_rows(const frisk_ref_desc* d, const void* A, const void* B, void* C,
                        const float* sa, const float* sb, int64_t m_begin, int64_t m_end,
                        int num_threads) {
  if (!valid_desc(d) || !A || !B || !C) return -1;
  if (d->use_scales && (!sa || !sb)) return -1;
  if (m_begin < 0 || m_end > d->M || m_begin > m_end) return -1;
  const int64_t N = d->N, K = d->K;
  int failed = 0;
#ifdef _OPENMP
  if (num_threads > 0) omp_set_num_threads(num_threads);
#else
  (void)num_threads;
#endif
#pragma omp parallel
  {
    float* arow = (float*)malloc(sizeof(float) * (size_t)K);
    float* acc = (float*)malloc(sizeof(float) * (size_t)N);
    double* acc64 = d->acc64 ? (double*)malloc(sizeof(double) * (size_t)N) : NULL;
    float* brow = (float*)malloc(sizeof(float) * (size_t)(d->transB ? K : N));
    if (!arow || !acc || !brow || (d->acc64 && !acc64)) {
#pragma omp atomic write
      failed = 1;
    } else {
#pragma omp for schedule(dynamic, 1)
      for (int64_t m = m_begin; m < m_end; ++m) {
        for (int64_t k = 0; k < K; ++k)
          arow[k] = decode_in(A, d->transA ? k * d->lda + m : m * d->lda + k, d->ab_type);
        if (d->transB) {
          /* B[k,n] at n*ldb + k: one dot product per output, k increasing */
          for (int64_t n = 0; n < N; ++n) {
            for (int64_t k = 0; k < K; ++k) brow[k] = decode_in(B, n * d->ldb + k, d->ab_type);
            if (d->acc64) {
              double s = 0.0;
              for (int64_t k = 0; k < K; ++k) s += (double)arow[k] * (double)brow[k];
              acc64[n] = s;
            } else {
              float s = 0.0f;
              for (int64_t k = 0; k < K; ++k) s += arow[k] * brow[k];
              acc[n] = s;
            }
          }
        } else {
          /* B[k,n] at k*ldb + n: rank-1 updates; every acc[n] still sums in increasing k */
          if (d->acc64) memset(acc64, 0, sizeof(double) * (size_t)N);
          else memset(acc, 0, sizeof(float) * (size_t)N);
          for (int64_t k = 0; k < K; ++k) {
            const float a = arow[k];
            for (int64_t n = 0; n < N; ++n) brow[n] = decode_in(B, k * d->ldb + n, d->ab_type);
            if (d->acc64) {
              for (int64_t n = 0; n < N; ++n) acc64[n] += (double)a * (double)brow[n];
            } else {
              for (int64_t n = 0; n < N; ++n) acc[n] += a * brow[n];
            }
          }
        }
        for (int64_t n = 0; n < N; ++n) {
          float v = d->acc64 ? (float)acc64[n] : acc[n];
          if (d->use_scales) v = v * sa[m] * sb[n];
          if (!d->clear_accum) {
            const int64_t ci = m * d->ldc + n;
            float old;
            switch (d->c_type) {
              case REF_F32: old = ((const float*)C)[ci]; break;
              case REF_F16: old = frisk_ref_decode_f16(((const uint16_t*)C)[ci]); break;
              default: old = frisk_ref_decode_bf16(((const uint16_t*)C)[ci]); break;
            }
            v += old;
          }
          store_out(C, m * d->ldc + n, d->c_type, v);
        }
      }
    }
    free(arow);
    free(acc);
    free(acc64);
    free(brow);
  }
  return failed ? -1 : 0;
}

int frisk_ref_gemm(const frisk_ref_desc* d, const void* A, const void* B, void* C, const float* sa,
                   const float* sb, int num_threads) {
  if (!d) return -1;
  return frisk_ref_gemm_rows(d, A, B, C, sa, sb, 0, d->M, num_threads);
}

int frisk_ref_max_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}
