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

/* ---------------------------------------------------------------------------
 * Register-blocked nests: what the reference's multi-level schedules produce.
 *
 * The reference's tuned schedules (Strategy "tile_oo" / "tile_pprprp_vr",
 * src/xtc/search/strategies.py:638-670,772-781) tile every axis twice, put the
 * innermost i/j tile inside the k loop, vectorize the innermost j tile and
 * unroll the innermost i tile: the i2 x j2 accumulator tile then lives in
 * vector registers for a whole k tile.  `pack_at` / `buffer_at`
 * (src/xtc/itf/schd/scheduler.py:174-215) copy the operand blocks of a tile
 * level into contiguous buffers.  The functions below are that nest written by
 * hand; (mc, nc, kc, micro) and (wt, nv) are the sample a search tunes.
 *
 *   tile(i, {i1: mc, i2: MR}); tile(j, {j1: nc, j2: NR}); tile(k, {k1: kc})
 *   interchange [i, j, k, j1.., i1.., k1, i2, j2]; parallelize [i, j]
 *   pack_at(k, A); pack_at(k, B); vectorize [j2]; unroll {i2: MR}
 * ------------------------------------------------------------------------- */
#include <stdlib.h>

#if defined(__AVX512F__)
#define VW 16
#elif defined(__AVX__)
#define VW 8
#else
#define VW 4
#endif
typedef float vf __attribute__((vector_size(VW * 4), aligned(4)));

int xtc_ref_vector_width(void) { return VW; }

/* acc[MR][NV] += Ap[k][MR] (x) Bp[k][NV*VW] over kc steps; C block updated in place. */
#define DEFINE_MICRO(MR, NV)                                                                  \
  static void micro_##MR##x##NV(const float* restrict Ap, const float* restrict Bp,           \
                                float* restrict Cb, int64_t ldc, int64_t kc, int first,       \
                                int64_t mr, int64_t nr) {                                     \
    vf acc[MR][NV];                                                                           \
    _Pragma("GCC unroll 16") for (int i = 0; i < MR; ++i)                                     \
        _Pragma("GCC unroll 8") for (int v = 0; v < NV; ++v) acc[i][v] = (vf){0};             \
    for (int64_t k = 0; k < kc; ++k) {                                                        \
      vf b[NV];                                                                               \
      _Pragma("GCC unroll 8") for (int v = 0; v < NV; ++v)                                    \
          b[v] = *(const vf*)(Bp + k * (NV * VW) + v * VW);                                   \
      _Pragma("GCC unroll 16") for (int i = 0; i < MR; ++i) {                                 \
        const float a = Ap[k * MR + i];                                                       \
        _Pragma("GCC unroll 8") for (int v = 0; v < NV; ++v) acc[i][v] += a * b[v];           \
      }                                                                                       \
    }                                                                                         \
    if (mr == MR && nr == NV * VW) {                                                          \
      _Pragma("GCC unroll 16") for (int i = 0; i < MR; ++i)                                   \
          _Pragma("GCC unroll 8") for (int v = 0; v < NV; ++v) {                              \
        vf* c = (vf*)(Cb + i * ldc + v * VW);                                                 \
        *c = first ? acc[i][v] : *c + acc[i][v];                                              \
      }                                                                                       \
    } else {                                                                                  \
      for (int64_t i = 0; i < mr; ++i)                                                        \
        for (int64_t j = 0; j < nr; ++j) {                                                    \
          const float x = acc[i][j / VW][j % VW];                                             \
          Cb[i * ldc + j] = first ? x : Cb[i * ldc + j] + x;                                  \
        }                                                                                     \
    }                                                                                         \
  }

DEFINE_MICRO(4, 1)
DEFINE_MICRO(6, 1)
DEFINE_MICRO(8, 1)
DEFINE_MICRO(12, 1)
DEFINE_MICRO(4, 2)
DEFINE_MICRO(6, 2)
DEFINE_MICRO(8, 2)
DEFINE_MICRO(12, 2)
DEFINE_MICRO(14, 2)
DEFINE_MICRO(4, 3)
DEFINE_MICRO(6, 3)
DEFINE_MICRO(8, 3)
DEFINE_MICRO(4, 4)
DEFINE_MICRO(6, 4)

typedef void (*micro_fn)(const float*, const float*, float*, int64_t, int64_t, int, int64_t, int64_t);
static const struct { int mr, nv; micro_fn fn; } MICROS[] = {
    {4, 1, micro_4x1},   {6, 1, micro_6x1},   {8, 1, micro_8x1}, {12, 1, micro_12x1},
    {4, 2, micro_4x2},   {6, 2, micro_6x2},   {8, 2, micro_8x2}, {12, 2, micro_12x2},
    {14, 2, micro_14x2}, {4, 3, micro_4x3},   {6, 3, micro_6x3}, {8, 3, micro_8x3},
    {4, 4, micro_4x4},   {6, 4, micro_6x4}};
#define N_MICROS ((int)(sizeof(MICROS) / sizeof(MICROS[0])))

int xtc_ref_micro_count(void) { return N_MICROS; }
/* rows and columns (in floats) of the register tile of micro-kernel `idx` */
int xtc_ref_micro_shape(int idx, int* rows, int* cols) {
  if (idx < 0 || idx >= N_MICROS) return 1;
  *rows = MICROS[idx].mr;
  *cols = MICROS[idx].nv * VW;
  return 0;
}

/* C = A * B with the two-level tiling above.  Returns 0, or 1 for a bad sample. */
int xtc_ref_matmul_blocked(const float* A, const float* B, float* C, int64_t M, int64_t N, int64_t K,
                           int64_t mc, int64_t nc, int64_t kc, int micro, int relu) {
  if (micro < 0 || micro >= N_MICROS || mc <= 0 || nc <= 0 || kc <= 0) return 1;
  const int MR = MICROS[micro].mr, NR = MICROS[micro].nv * VW;
  const micro_fn kern = MICROS[micro].fn;
  mc = (mc + MR - 1) / MR * MR;
  nc = (nc + NR - 1) / NR * NR;
  const int64_t nti = (M + mc - 1) / mc, ntj = (N + nc - 1) / nc;
  int bad = 0;
#pragma omp parallel
  {
    float* Ap = aligned_alloc(64, (size_t)(mc * kc) * sizeof(float));
    float* Bp = aligned_alloc(64, (size_t)(kc * nc) * sizeof(float));
    if (!Ap || !Bp) {
#pragma omp atomic write
      bad = 1;
    }
#pragma omp barrier
    if (!bad) {
#pragma omp for collapse(2) schedule(dynamic)
      for (int64_t it = 0; it < nti; ++it) {
        for (int64_t jt = 0; jt < ntj; ++jt) {
          const int64_t i0 = it * mc, ib = min64(M - i0, mc);
          const int64_t j0 = jt * nc, jb = min64(N - j0, nc);
          for (int64_t k0 = 0; k0 < K; k0 += kc) {
            const int64_t kb = min64(K - k0, kc);
            /* pack_at(k, B): NR-wide column panels, k-major inside a panel, zero padded */
            for (int64_t jr = 0; jr < jb; jr += NR) {
              float* dst = Bp + jr * kb;
              const int64_t w = min64(NR, jb - jr);
              for (int64_t k = 0; k < kb; ++k) {
                const float* src = B + (k0 + k) * N + j0 + jr;
                for (int64_t j = 0; j < w; ++j) dst[k * NR + j] = src[j];
                for (int64_t j = w; j < NR; ++j) dst[k * NR + j] = 0.f;
              }
            }
            /* pack_at(k, A): MR-row panels, k-major inside a panel, zero padded */
            for (int64_t ir = 0; ir < ib; ir += MR) {
              float* dst = Ap + ir * kb;
              const int64_t h = min64(MR, ib - ir);
              for (int64_t i = 0; i < h; ++i) {
                const float* src = A + (i0 + ir + i) * K + k0;
                for (int64_t k = 0; k < kb; ++k) dst[k * MR + i] = src[k];
              }
              for (int64_t i = h; i < MR; ++i)
                for (int64_t k = 0; k < kb; ++k) dst[k * MR + i] = 0.f;
            }
            for (int64_t jr = 0; jr < jb; jr += NR)
              for (int64_t ir = 0; ir < ib; ir += MR)
                kern(Ap + ir * kb, Bp + jr * kb, C + (i0 + ir) * N + j0 + jr, N, kb, k0 == 0,
                     min64(MR, ib - ir), min64(NR, jb - jr));
          }
        }
      }
    }
    free(Ap);
    free(Bp);
  }
  if (bad) return 1;
  if (relu) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < M * N; ++i) C[i] = C[i] > 0.f ? C[i] : 0.f;
  }
  return 0;
}

/* conv2d with a register tile of WT output pixels x NV vectors of filters:
 *   tile(w, {w1: WT}); tile(f, {f1: NV*VW}); interchange [b, h, w, f, r, s, c, w1, f1];
 *   parallelize [b, h]; vectorize [f1]; unroll {w1: WT}. */
#define DEFINE_CONV(WT, NV)                                                                   \
  static void conv_##WT##x##NV(const float* restrict X, const float* restrict Wt,             \
                               float* restrict Y, int64_t W, int64_t C, int64_t R, int64_t S, \
                               int64_t F, int64_t sw, int64_t wn, int64_t fn, int relu) {     \
    /* X: first pixel of the row under tap (0,0); Y: first output pixel; Wt: + f0 */          \
    vf acc[WT][NV];                                                                           \
    _Pragma("GCC unroll 16") for (int i = 0; i < WT; ++i)                                     \
        _Pragma("GCC unroll 8") for (int v = 0; v < NV; ++v) acc[i][v] = (vf){0};             \
    for (int64_t r = 0; r < R; ++r)                                                           \
      for (int64_t s = 0; s < S; ++s) {                                                       \
        const float* x = X + (r * W + s) * C;                                                 \
        const float* w = Wt + (r * S + s) * C * F;                                            \
        for (int64_t c = 0; c < C; ++c) {                                                     \
          vf b[NV];                                                                           \
          _Pragma("GCC unroll 8") for (int v = 0; v < NV; ++v)                                \
              b[v] = *(const vf*)(w + c * F + v * VW);                                        \
          _Pragma("GCC unroll 16") for (int i = 0; i < WT; ++i) {                             \
            const float a = i < wn ? x[i * sw * C + c] : 0.f;                                 \
            _Pragma("GCC unroll 8") for (int v = 0; v < NV; ++v) acc[i][v] += a * b[v];       \
          }                                                                                   \
        }                                                                                     \
      }                                                                                       \
    for (int64_t i = 0; i < wn; ++i)                                                          \
      for (int64_t j = 0; j < fn; ++j) {                                                      \
        float v = acc[i][j / VW][j % VW];                                                     \
        if (relu && v < 0.f) v = 0.f;                                                         \
        Y[i * F + j] = v;                                                                     \
      }                                                                                       \
  }
DEFINE_CONV(2, 4)
DEFINE_CONV(4, 4)
DEFINE_CONV(6, 4)
DEFINE_CONV(4, 2)
DEFINE_CONV(7, 2)
DEFINE_CONV(8, 2)
DEFINE_CONV(14, 2)
DEFINE_CONV(8, 1)
DEFINE_CONV(14, 1)
typedef void (*conv_fn)(const float*, const float*, float*, int64_t, int64_t, int64_t, int64_t,
                        int64_t, int64_t, int64_t, int64_t, int);
static const struct { int wt, nv; conv_fn fn; } CONVS[] = {
    {2, 4, conv_2x4}, {4, 4, conv_4x4}, {6, 4, conv_6x4},   {4, 2, conv_4x2},  {7, 2, conv_7x2},
    {8, 2, conv_8x2}, {14, 2, conv_14x2}, {8, 1, conv_8x1}, {14, 1, conv_14x1}};
#define N_CONVS ((int)(sizeof(CONVS) / sizeof(CONVS[0])))
int xtc_ref_conv_micro_count(void) { return N_CONVS; }
int xtc_ref_conv_micro_shape(int idx, int* pixels, int* filters) {
  if (idx < 0 || idx >= N_CONVS) return 1;
  *pixels = CONVS[idx].wt;
  *filters = CONVS[idx].nv * VW;
  return 0;
}

int xtc_ref_conv2d_blocked(const float* X, const float* Wt, float* Y, int64_t B, int64_t H, int64_t W,
                           int64_t C, int64_t R, int64_t S, int64_t F, int64_t sh, int64_t sw,
                           int micro, int relu) {
  if (micro < 0 || micro >= N_CONVS) return 1;
  const int WT = CONVS[micro].wt, FT = CONVS[micro].nv * VW;
  const conv_fn kern = CONVS[micro].fn;
  const int64_t OH = (H - R) / sh + 1, OW = (W - S) / sw + 1;
  /* the kernel reads whole vectors of filters: pad the filter bank to a multiple of FT */
  const int64_t Fp = (F + FT - 1) / FT * FT;
  float* Wp = (float*)Wt;
  if (Fp != F) {
    Wp = aligned_alloc(64, (size_t)(R * S * C * Fp) * sizeof(float));
    if (!Wp) return 1;
    for (int64_t q = 0; q < R * S * C; ++q) {
      for (int64_t f = 0; f < F; ++f) Wp[q * Fp + f] = Wt[q * F + f];
      for (int64_t f = F; f < Fp; ++f) Wp[q * Fp + f] = 0.f;
    }
  }
#pragma omp parallel for collapse(2) schedule(static)
  for (int64_t b = 0; b < B; ++b)
    for (int64_t h = 0; h < OH; ++h)
      for (int64_t w0 = 0; w0 < OW; w0 += WT)
        for (int64_t f0 = 0; f0 < F; f0 += FT) {
          const float* x = X + ((b * H + h * sh) * W + w0 * sw) * C;
          float* y = Y + ((b * OH + h) * OW + w0) * F + f0;
          /* the kernel's weight pitch is its F argument */
          if (Fp == F) {
            kern(x, Wt + f0, y, W, C, R, S, F, sw, min64(WT, OW - w0), min64(FT, F - f0), relu);
          } else {
            float tmp[16 * 64];
            const int64_t wn = min64(WT, OW - w0), fn = min64(FT, F - f0);
            kern(x, Wp + f0, tmp, W, C, R, S, Fp, sw, wn, FT, relu);
            for (int64_t i = 0; i < wn; ++i)
              for (int64_t j = 0; j < fn; ++j) y[i * F + j] = tmp[i * Fp + j];
          }
        }
  if (Wp != Wt) free(Wp);
  return 0;
}

/* Peak fused-multiply-add rate of the host cores in FMA/s (all OpenMP threads):
 * twelve independent register-resident vector FMA chains per thread, the CPU twin of
 * the reference's probe (src/xtc/csrcs/runtimes/host/evaluate_flops.c:461-495). */
#if VW == 16
#define KEEP(v) __asm__ volatile("" : "+v"(v))
#else
#define KEEP(v) __asm__ volatile("" : "+x"(v))
#endif
#define CHAINS(OP) OP(a0) OP(a1) OP(a2) OP(a3) OP(a4) OP(a5) OP(a6) OP(a7) OP(a8) OP(a9) OP(a10) OP(a11)
double xtc_ref_peak_fma(void) {
  const int64_t iters = 4000000;
  double t_best = 1e30;
  int threads = 1;
  for (int rep = 0; rep < 3; ++rep) {
    double t0 = 0, t1 = 0;
#pragma omp parallel
    {
      const vf x = (vf){0} + 0.999f, y = (vf){0} + 1e-6f;
#define INIT(v) vf v = x;
      CHAINS(INIT)
#pragma omp barrier
#pragma omp master
      {
#ifdef _OPENMP
        t0 = omp_get_wtime();
        threads = omp_get_num_threads();
#endif
      }
      for (int64_t it = 0; it < iters; ++it) {
        /* the empty asm makes every value needed, in a register, every iteration */
#define STEP(v) v = v * x + y; KEEP(v);
        CHAINS(STEP)
      }
#pragma omp barrier
#pragma omp master
      {
#ifdef _OPENMP
        t1 = omp_get_wtime();
#endif
      }
    }
    if (t1 - t0 > 0 && t1 - t0 < t_best) t_best = t1 - t0;
  }
  return (double)threads * (double)iters * 12.0 * VW / t_best;
}
