/*
 * CPU restatement of the loop nests the reference's MLIR llvmir backend
 * generates for the hot-path operators -- TEST / BASELINE INFRASTRUCTURE, not
 * product code.  Only tests/, __graft_entry__.smoke() and bench.py's
 * cpu_baseline / reference legs may use it.
 *
 * The reference lowers each node to linalg ops and then to scalar loops that a
 * schedule tiles, interchanges, parallelises (OpenMP) and vectorises; LLVM
 * compiles them with -O2 --fp-contract=fast (src/xtc/utils/ext_tools.py:48-69).
 * The functions below are those nests written by hand in C with the schedule's
 * tile sizes as arguments:
 *   matmul : linalg.fill(0) + linalg.matmul, src/xtc/backends/mlir/MlirOps.py:189-270
 *   conv2d : linalg.fill(0) + 7-D linalg.generic (b,h,w,f,r,s,c), MlirOps.py:331-420
 *   relu   : arith.maximumf(x, 0) over the flattened tensor, MlirOps.py:459-557
 *   pad    : linalg.fill(constant) + linalg.copy into the interior, MlirOps.py:718-735
 *   transpose : src/xtc/graphs/xtc/operators.py:757-787 (no MLIR lowering exists)
 * Build: see oracle/Makefile (cc -O3 -march=native -ffp-contract=fast -fopenmp,
 * the flags of src/xtc/targets/host/HostCEvaluator.py:40-63 plus OpenMP).
 */
#include <stddef.h>
#include <stdint.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

static inline int64_t min64(int64_t a, int64_t b) { return a < b ? a : b; }

int xtc_ref_max_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/* C[M,N] = A[M,K] * B[K,N], schedule: i tiled by ti (parallel), k tiled by tk,
 * j innermost and vectorised -- the reference's "tile, parallelize outer i,
 * vectorize inner j" family (e.g. tests/pytest/mlir/test_mlir_impl.py:29-45). */
void xtc_ref_matmul(const float* A, const float* B, float* C, int64_t M, int64_t N, int64_t K,
                    int64_t ti, int64_t tj, int64_t tk, int relu) {
  if (ti <= 0) ti = 64;
  if (tj <= 0) tj = N;
  if (tk <= 0) tk = 64;
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < M; ++i) memset(C + i * N, 0, (size_t)N * sizeof(float));
  const int64_t nti = (M + ti - 1) / ti, ntj = (N + tj - 1) / tj;
#pragma omp parallel for collapse(2) schedule(dynamic)
  for (int64_t it = 0; it < nti; ++it) {
    for (int64_t jt = 0; jt < ntj; ++jt) {
      const int64_t i0 = it * ti, i1 = min64(M, i0 + ti);
      const int64_t j0 = jt * tj, j1 = min64(N, j0 + tj);
      for (int64_t k0 = 0; k0 < K; k0 += tk) {
        const int64_t k1 = min64(K, k0 + tk);
        for (int64_t i = i0; i < i1; ++i) {
          float* c = C + i * N;
          for (int64_t k = k0; k < k1; ++k) {
            const float a = A[i * K + k];
            const float* b = B + k * N;
#pragma omp simd
            for (int64_t j = j0; j < j1; ++j) c[j] += a * b[j];
          }
        }
      }
    }
  }
  if (relu) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < M * N; ++i) C[i] = C[i] > 0.f ? C[i] : 0.f;
  }
}

/* Y[B,OH,OW,F] over X[B,H,W,C] (already padded) and Wt[R,S,C,F]; loop order
 * b,h,w (parallel) / r,s,c / f vectorised. */
void xtc_ref_conv2d(const float* X, const float* Wt, float* Y, int64_t B, int64_t H, int64_t W,
                    int64_t C, int64_t R, int64_t S, int64_t F, int64_t sh, int64_t sw, int relu) {
  const int64_t OH = (H - R) / sh + 1, OW = (W - S) / sw + 1;
#pragma omp parallel for collapse(2) schedule(static)
  for (int64_t b = 0; b < B; ++b) {
    for (int64_t h = 0; h < OH; ++h) {
      for (int64_t w = 0; w < OW; ++w) {
        float* y = Y + ((b * OH + h) * OW + w) * F;
        for (int64_t f = 0; f < F; ++f) y[f] = 0.f;
        for (int64_t r = 0; r < R; ++r)
          for (int64_t s = 0; s < S; ++s) {
            const float* x = X + ((b * H + h * sh + r) * W + w * sw + s) * C;
            const float* wt = Wt + (r * S + s) * C * F;
            for (int64_t c = 0; c < C; ++c) {
              const float xv = x[c];
#pragma omp simd
              for (int64_t f = 0; f < F; ++f) y[f] += xv * wt[c * F + f];
            }
          }
        if (relu)
          for (int64_t f = 0; f < F; ++f) y[f] = y[f] > 0.f ? y[f] : 0.f;
      }
    }
  }
}

void xtc_ref_relu(const float* X, float* Y, int64_t n, float threshold) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) Y[i] = X[i] > threshold ? X[i] : threshold;
}

/* 4-D pad of axes 1 and 2 (NHWC spatial pad): fill, then copy the interior rows. */
void xtc_ref_pad_hw(const float* X, float* Y, int64_t B, int64_t H, int64_t W, int64_t C,
                    int64_t pt, int64_t pb, int64_t pl, int64_t pr, float value) {
  const int64_t OH = H + pt + pb, OW = W + pl + pr;
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < B * OH * OW * C; ++i) Y[i] = value;
#pragma omp parallel for collapse(2) schedule(static)
  for (int64_t b = 0; b < B; ++b)
    for (int64_t h = 0; h < H; ++h)
      memcpy(Y + ((b * OH + h + pt) * OW + pl) * C, X + (b * H + h) * W * C,
             (size_t)(W * C) * sizeof(float));
}

/* Y[C,R] = X[R,C]^T, 32x32 blocked. */
void xtc_ref_transpose2d(const float* X, float* Y, int64_t R, int64_t C) {
  const int64_t T = 32;
#pragma omp parallel for collapse(2) schedule(static)
  for (int64_t r0 = 0; r0 < R; r0 += T)
    for (int64_t c0 = 0; c0 < C; c0 += T) {
      const int64_t r1 = min64(R, r0 + T), c1 = min64(C, c0 + T);
      for (int64_t c = c0; c < c1; ++c)
        for (int64_t r = r0; r < r1; ++r) Y[c * R + r] = X[r * C + c];
    }
}
