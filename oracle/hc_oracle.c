/*
 * CPU restatement of Honeycrisp's CPUBackend matrix product.  TEST INFRASTRUCTURE ONLY:
 * the checker that the CUDA kernels are compared with, and the timed CPU baseline.
 * Nothing in the shipped library links, loads or calls this file.
 *
 * What it follows in the reference (paths inside the Honeycrisp project):
 *   Sources/Honeycrisp/BackendCPU.swift:1234-1313   batchedMatmul: dispatch, index maps, loop
 *   Sources/Honeycrisp/BackendCPU.swift:1222-1232   matmul = batchedMatmul(matrixCount: 1)
 *   Sources/Honeycrisp/BackendCPU.swift:2018-2058   readBuffer / writeBuffer: widen to Float,
 *                                                   compute, narrow once on the way out
 *   Sources/Honeycrisp/TensorElement.swift:262-277,325-338  fp16<->fp32 through vImage planar
 *                                                   conversion (widening exact, narrowing RNE)
 *
 * Parity status: PINNED on the reference's own known-answer tests for this path
 * (Sources/HCTestUtils/BackendTests.swift:684-783), which the test-suite replays against
 * this file.  The reference cannot be compiled on Linux (Swift + Apple Accelerate), so
 * there is no run of the reference itself behind these functions.  One call in the
 * reference is closed source: vDSP_mmul (BackendCPU.swift:1256, fp32 with no transposes).
 * Its stand-in here is a caller-supplied row-major sgemm (OpenBLAS cblas_sgemm) with the
 * reference's argument mapping; summation order inside Accelerate is unknown, so that one
 * case is a tolerance comparison, never bitwise.
 *
 * Build: gcc -O2 -ffp-contract=off -fopenmp -shared -fPIC (see oracle/build.py).
 * -ffp-contract=off matters: the reference computes `acc = acc + a * b` with two roundings.
 */
#include <stdint.h>
#include <stddef.h>
#include <string.h>
#include <stdlib.h>

/* ---- fp16 <-> fp32, bit-level (IEEE binary16; widening exact, narrowing RNE, overflow -> inf) */

static float half_to_float(uint16_t h) {
  uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1fu;
  uint32_t man = h & 0x3ffu;
  uint32_t bits;
  if (exp == 0) {
    if (man == 0) {
      bits = sign;
    } else { /* subnormal: renormalise */
      int e = -1;
      do {
        man <<= 1;
        e++;
      } while ((man & 0x400u) == 0);
      man &= 0x3ffu;
      bits = sign | ((uint32_t)(127 - 15 - e) << 23) | (man << 13);
    }
  } else if (exp == 31) {
    bits = sign | 0x7f800000u | (man << 13);
  } else {
    bits = sign | ((exp + 127 - 15) << 23) | (man << 13);
  }
  float f;
  memcpy(&f, &bits, 4);
  return f;
}

static uint16_t float_to_half(float f) {
  uint32_t x;
  memcpy(&x, &f, 4);
  uint32_t sign = (x >> 16) & 0x8000u;
  uint32_t absx = x & 0x7fffffffu;
  if (absx >= 0x7f800000u) { /* inf / nan */
    uint32_t man = absx & 0x7fffffu;
    return (uint16_t)(sign | 0x7c00u | (man ? (0x200u | (man >> 13)) : 0));
  }
  if (absx >= 0x477ff000u) { /* >= 65520 rounds to inf */
    return (uint16_t)(sign | 0x7c00u);
  }
  if (absx < 0x38800000u) { /* below the smallest normal half: subnormal or zero */
    if (absx < 0x33000000u) { /* < 2^-25 rounds to zero (2^-25 itself ties to even = 0) */
      return (uint16_t)sign;
    }
    uint32_t exp = absx >> 23;
    uint32_t man = (absx & 0x7fffffu) | 0x800000u;
    uint32_t shift = 126 - exp; /* 14..24: bits dropped from the 24-bit significand */
    uint32_t half_man = man >> shift;
    uint32_t rem = man & ((1u << shift) - 1);
    uint32_t halfway = 1u << (shift - 1);
    if (rem > halfway || (rem == halfway && (half_man & 1u))) half_man++;
    return (uint16_t)(sign | half_man);
  }
  uint32_t exp = (absx >> 23) - 127 + 15;
  uint32_t man = absx & 0x7fffffu;
  uint32_t half = (exp << 10) | (man >> 13);
  uint32_t rem = man & 0x1fffu;
  if (rem > 0x1000u || (rem == 0x1000u && (half & 1u))) half++; /* carries into exp correctly */
  return (uint16_t)(sign | half);
}

void hc_oracle_half_to_float(const uint16_t *in, float *out, int64_t n) {
  for (int64_t i = 0; i < n; i++) out[i] = half_to_float(in[i]);
}

void hc_oracle_float_to_half(const float *in, uint16_t *out, int64_t n) {
  for (int64_t i = 0; i < n; i++) out[i] = float_to_half(in[i]);
}

/* ---- the literal loop (BackendCPU.swift:1266-1300) on Float arrays ----------------------
 * Rows [row_begin, row_end) of every matrix are computed; the full call passes 0, rows.
 * Restricting rows only selects which outputs are produced: each output element is an
 * independent sequential sum, so a row sample is bit-identical to the same rows of a full run.
 * The OpenMP loop splits those independent rows over threads for the timed baseline; the
 * reference itself runs them on one worker thread (BackendCPU.swift:226,235-248). */
static void loop_f32(int64_t matrix_count, const float *a, int trans_a, const float *b,
                     int trans_b, int trans_out, int64_t rows, int64_t inner, int64_t cols,
                     float *c, int64_t row_begin, int64_t row_end, int threads) {
  if (threads < 1) threads = 1;
  for (int64_t mat = 0; mat < matrix_count; mat++) {
    const float *am = a + mat * rows * inner;
    const float *bm = b + mat * cols * inner;
    float *cm = c + mat * rows * cols;
#pragma omp parallel for num_threads(threads) schedule(static)
    for (int64_t i = row_begin; i < row_end; i++) {
      for (int64_t j = 0; j < cols; j++) {
        float acc = 0.0f;
        for (int64_t k = 0; k < inner; k++) {
          float av = trans_a ? am[i + k * rows] : am[i * inner + k];
          float bv = trans_b ? bm[k + j * inner] : bm[k * cols + j];
          acc = acc + av * bv;
        }
        if (trans_out) {
          cm[i + j * rows] = acc;
        } else {
          cm[i * cols + j] = acc;
        }
      }
    }
  }
}

/* Row-major sgemm supplied by the caller (cblas_sgemm signature, LP64 ints). */
typedef void (*hc_sgemm_fn)(int order, int ta, int tb, int m, int n, int k, float alpha,
                            const float *a, int lda, const float *b, int ldb, float beta,
                            float *c, int ldc);
/* ILP64 flavour (scipy_cblas_sgemm64_ in numpy's bundled OpenBLAS). */
typedef void (*hc_sgemm64_fn)(int order, int ta, int tb, int64_t m, int64_t n, int64_t k,
                              float alpha, const float *a, int64_t lda, const float *b,
                              int64_t ldb, float beta, float *c, int64_t ldc);

enum { kRowMajor = 101, kNoTrans = 111 };

/*
 * float32 entry point.  Returns 0 on success, 1 if the fast path was requested without an
 * sgemm.  `sgemm`/`sgemm_ilp64`: at most one non-null; both null forces the literal loop even
 * for the no-transpose case (used to compare the two CPU paths with each other).
 *
 * Dispatch as BackendCPU.swift:1245: no flags and float32 -> one library GEMM per matrix,
 * vDSP_mmul(A,1,B,1,C,1,rows,cols,inner) == sgemm(RowMajor,N,N,rows,cols,inner,1,A,inner,B,cols,0,C,cols).
 */
int hc_oracle_batched_matmul_f32(int64_t matrix_count, const float *a, int trans_a,
                                 const float *b, int trans_b, int trans_out, int64_t rows,
                                 int64_t inner, int64_t cols, float *c, void *sgemm,
                                 void *sgemm_ilp64, int use_library_fast_path) {
  if (!trans_a && !trans_b && !trans_out && use_library_fast_path) {
    if (!sgemm && !sgemm_ilp64) return 1;
    for (int64_t i = 0; i < matrix_count; i++) {
      const float *x = a + i * rows * inner;
      const float *y = b + i * inner * cols;
      float *z = c + i * rows * cols;
      if (sgemm) {
        ((hc_sgemm_fn)sgemm)(kRowMajor, kNoTrans, kNoTrans, (int)rows, (int)cols, (int)inner,
                             1.0f, x, (int)inner, y, (int)cols, 0.0f, z, (int)cols);
      } else {
        ((hc_sgemm64_fn)sgemm_ilp64)(kRowMajor, kNoTrans, kNoTrans, rows, cols, inner, 1.0f, x,
                                     inner, y, cols, 0.0f, z, cols);
      }
    }
    return 0;
  }
  loop_f32(matrix_count, a, trans_a, b, trans_b, trans_out, rows, inner, cols, c, 0, rows, 1);
  return 0;
}

/*
 * float16 entry point: widen whole operands to Float (readBuffer), run the loop into a
 * Float output (writeBuffer's temporary), narrow once (arrayToPointer -> convertFloatToHalf).
 * Returns 0, or 2 if the temporaries cannot be allocated.
 */
int hc_oracle_batched_matmul_f16(int64_t matrix_count, const uint16_t *a, int trans_a,
                                 const uint16_t *b, int trans_b, int trans_out, int64_t rows,
                                 int64_t inner, int64_t cols, uint16_t *c) {
  int64_t na = matrix_count * rows * inner, nb = matrix_count * inner * cols,
          nc = matrix_count * rows * cols;
  float *fa = (float *)malloc(sizeof(float) * (size_t)(na ? na : 1));
  float *fb = (float *)malloc(sizeof(float) * (size_t)(nb ? nb : 1));
  float *fc = (float *)malloc(sizeof(float) * (size_t)(nc ? nc : 1));
  if (!fa || !fb || !fc) {
    free(fa);
    free(fb);
    free(fc);
    return 2;
  }
  hc_oracle_half_to_float(a, fa, na);
  hc_oracle_half_to_float(b, fb, nb);
  loop_f32(matrix_count, fa, trans_a, fb, trans_b, trans_out, rows, inner, cols, fc, 0, rows, 1);
  hc_oracle_float_to_half(fc, c, nc);
  free(fa);
  free(fb);
  free(fc);
  return 0;
}

/*
 * Row-sampled variants for large shapes and for the timed baseline: operands are already
 * Float (the caller widens fp16 once, outside the timed region or inside it as it chooses);
 * only rows [row_begin,row_end) of each matrix of `c` (a full-size Float output) are written.
 */
void hc_oracle_loop_rows_f32(int64_t matrix_count, const float *a, int trans_a, const float *b,
                             int trans_b, int trans_out, int64_t rows, int64_t inner,
                             int64_t cols, float *c, int64_t row_begin, int64_t row_end,
                             int threads) {
  loop_f32(matrix_count, a, trans_a, b, trans_b, trans_out, rows, inner, cols, c, row_begin,
           row_end, threads);
}
