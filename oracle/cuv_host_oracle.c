/*
 * CPU oracle for the DIA sparse hot path of CUV.
 *
 * TEST INFRASTRUCTURE ONLY.  This file restates, in plain C, the algorithm of
 * CUV's host_memory_space code for the DIA path.  It is the checker the CUDA
 * kernels are compared with and the CPU baseline that is timed beside them.
 * Nothing on the product path links, loads or calls it.
 *
 * Every function cites the reference file:line it follows (paths relative to
 * the CUV source tree).  Arithmetic is fp32 in the reference's operation
 * order; build with -ffp-contract=off so no multiply-add is fused.
 *
 * Parity status: the reference pins this path only through parametric test
 * fixtures (DIA result == dense result on `sequence`-filled inputs,
 * src/tests/spmv.cpp:65-143, src/tests/densedense_to_dia.cpp:66-197,
 * src/tests/dia_mat.cpp:111-132, src/tests/matrix_op.cpp:858-924).  Those
 * fixtures are rebuilt from their definitions in tests/golden/ and this oracle
 * is checked against them.  prod with row_fact > 1 and densedense_to_dia with
 * non-default factors are not pinned by any reference test; for those the
 * oracle is checked only against a float64 dense computation.
 *
 * Threading: optional pthreads split over batch columns (prod, reduce over
 * the contiguous axis) or over diagonals / output ranges (densedense_to_dia,
 * reduce over the strided axis).  Each output's summation order is unchanged
 * by the split, so results are bit-identical to one thread.
 */
#include <limits.h>
#include <math.h>
#include <float.h>
#include <pthread.h>
#include <stdlib.h>
#include <string.h>

#define ORACLE_API __attribute__((visibility("default")))

static inline int imax(int a, int b) { return a > b ? a : b; }
static inline int imin(int a, int b) { return a < b ? a : b; }

/* ------------------------------------------------------------------------ */
/* generic range-splitting thread pool                                        */
/* ------------------------------------------------------------------------ */
typedef void (*range_fn)(void *ctx, long lo, long hi);
typedef struct { range_fn fn; void *ctx; long lo, hi; } range_job;

static void *range_thread(void *p)
{
    range_job *j = (range_job *)p;
    j->fn(j->ctx, j->lo, j->hi);
    return NULL;
}

static void parallel_ranges(range_fn fn, void *ctx, long n, int nthreads)
{
    if (nthreads <= 1 || n <= 1) { fn(ctx, 0, n); return; }
    if (nthreads > n) nthreads = (int)n;
    pthread_t *th = (pthread_t *)malloc(sizeof(pthread_t) * nthreads);
    range_job *jobs = (range_job *)malloc(sizeof(range_job) * nthreads);
    for (int t = 0; t < nthreads; t++) {
        jobs[t].fn = fn; jobs[t].ctx = ctx;
        jobs[t].lo = n * t / nthreads;
        jobs[t].hi = n * (t + 1) / nthreads;
        pthread_create(&th[t], NULL, range_thread, &jobs[t]);
    }
    for (int t = 0; t < nthreads; t++) pthread_join(th[t], NULL);
    free(th); free(jobs);
}

/* ------------------------------------------------------------------------ */
/* DIA addressing                                                             */
/* ------------------------------------------------------------------------ */

/* Index into the value vector of matrix cell (i,j), or -1 when the diagonal
 * j - i/rf is not stored.  Follows basics/dia_matrix.hpp:228-251: the diagonal
 * is k = j - i/rf (integer division), its slot is the position of k in the
 * user-ordered offset list (the LAST position if k occurs twice, as
 * post_update_offsets overwrites, dia_matrix.hpp:181-185), the cell is
 * slot*stride + i. */
ORACLE_API long oracle_dia_cell_index(int h, int w, int rf, int stride, int nd,
                                      const int *offsets, int i, int j)
{
    (void)h; (void)w;
    int k = j - i / rf;
    int slot = -1;
    for (int s = 0; s < nd; s++) if (offsets[s] == k) slot = s;
    if (slot < 0) return -1;
    return (long)slot * stride + i;
}

/* dense(i,j) <- dia(i,j), column-major dense with leading dimension h.
 * Follows convert/convert.cu:42-66: zero-fill, then per diagonal walk
 * j from max(0,o), i from rf*max(0,-o), rf rows per column, reading each
 * cell through dia_matrix::operator() (dia_matrix.hpp:236-243). */
ORACLE_API void oracle_dia_to_dense(float *dense, int h, int w, int rf, int stride,
                                    int nd, const int *offsets, const float *vals)
{
    memset(dense, 0, sizeof(float) * (size_t)h * w);
    for (int oi = 0; oi < nd; oi++) {
        int o = offsets[oi];
        int j = imax(0, o);
        int i = rf * imax(0, -o);
        for (; i < h && j < w; j++) {
            for (int k = 0; k < rf; k++, i++) {
                if (i >= h) break; /* the reference would index past the end when h % rf != 0 */
                long c = oracle_dia_cell_index(h, w, rf, stride, nd, offsets, i, j);
                dense[(size_t)j * h + i] = c < 0 ? 0.f : vals[c];
            }
        }
    }
}

/* ------------------------------------------------------------------------ */
/* prod(C, A_dia, B, transA, 'n', factAB, factC)                              */
/* ------------------------------------------------------------------------ */

/* One column: follows spmv_impl::spmv host, matrix_ops/spmv.cu:145-200.
 * The pre-pass (dst = 0 or dst *= factC, :153-156), the per-diagonal start
 * rows/columns and counts (:165-169, :186-189) and the update expression
 * `*y += factAv * *d * *x` (:176, :196; evaluated left to right, so
 * (factAv*d)*x, a separate multiply and add) are kept verbatim in meaning. */
static void spmv_host(float *dst, const float *vals, const int *offsets, int nd,
                      int h, int w, int stride, int rf, const float *v,
                      char transA, float factAv, float factC)
{
    int max_dst = (transA == 't') ? w : h;
    if (factC == 0.f) for (int i = 0; i < max_dst; i++) dst[i] = 0;
    else              for (int i = 0; i < max_dst; i++) dst[i] = dst[i] * factC;
    if (transA == 't') {
        for (int i = 0; i < nd; i++) {
            int k = offsets[i];
            int i_start = imax(0, k);
            int j_start = rf * imax(0, -k);
            int N = imin((h - j_start) / rf, w - i_start);
            const float *d_ = vals + (size_t)i * stride + j_start;
            const float *x_ = v + j_start;
            float *y_ = dst + i_start;
            for (int n = 0; n < N; n++, y_++)
                for (int l = 0; l < rf; l++, x_++, d_++)
                    *y_ += factAv * *d_ * *x_;
        }
    } else {
        for (int i = 0; i < nd; i++) {
            int k = offsets[i];
            int i_start = rf * imax(0, -k);
            int j_start = imax(0, k);
            int N = imin(h - i_start, rf * (w - j_start));
            const float *d_ = vals + (size_t)i * stride + i_start;
            const float *x_ = v + j_start;
            float *y_ = dst + i_start;
            for (int n = 0; n < N; n++)
                *y_++ += factAv * *d_++ * x_[n / rf];
        }
    }
}

typedef struct {
    float *C; const float *vals; const int *offsets; int nd, h, w, stride, rf;
    const float *B; int ldb, ldc; char transA; float factAB, factC;
} prod_ctx;

static void prod_range(void *p, long lo, long hi)
{
    prod_ctx *c = (prod_ctx *)p;
    for (long col = lo; col < hi; col++)
        spmv_host(c->C + (size_t)col * c->ldc, c->vals, c->offsets, c->nd, c->h, c->w,
                  c->stride, c->rf, c->B + (size_t)col * c->ldb, c->transA, c->factAB, c->factC);
}

/* Column loop of prod host, matrix_ops/spmv.cu:203-220: one spmv per batch
 * column.  B is rows_B x ncols and C is rows_C x ncols, both column-major
 * with leading dimensions ldb / ldc.  Returns 0, or -1 for the argument
 * errors the reference asserts on (transB is not modelled: only 'n' exists). */
ORACLE_API int oracle_prod_dia(float *C, int ldc, const float *vals, const int *offsets,
                               int nd, int h, int w, int stride, int rf,
                               const float *B, int ldb, int ncols, char transA,
                               float factAB, float factC, int nthreads)
{
    if (transA != 'n' && transA != 't') return -1;
    if (rf <= 0 || stride < h) return -1;
    prod_ctx c = { C, vals, offsets, nd, h, w, stride, rf, B, ldb, ldc, transA, factAB, factC };
    parallel_ranges(prod_range, &c, ncols, nthreads);
    return 0;
}

/* ------------------------------------------------------------------------ */
/* densedense_to_dia                                                          */
/* ------------------------------------------------------------------------ */

typedef struct {
    float *Cv; const int *offsets; int nd, h, w, stride, rf;
    const float *A; int lda; const float *B; int ldb; int ncols;
    float factAB, factC; int literal;
} dd_ctx;

/* One diagonal at a time.  The raw sum follows the host loop,
 * matrix_ops/densedense_to_sparse.cu:217-251: row_start = rf*max(0,-k),
 * col_start = max(0,k), N = min(h-row_start, rf*(w-col_start)), and for every
 * batch column in order d[row_start+n] += A[row_start+n,b] * B[col_start+n/rf,b].
 *
 * literal != 0: exactly the host code, which accumulates onto the existing
 *   diagonal and ignores factAB/factC (:242-249).
 * literal == 0: the documented contract C = factC*C + factAB*(A*B^T)|dia
 *   (densedense_to_sparse.hpp:108-121) as the device kernel evaluates it
 *   (densedense_to_sparse.cu:104-119): the batch sum starts from 0, then
 *   factC*C_old + factAB*sum is stored (C_old is not read when factC == 0,
 *   the product by factAB is skipped when factAB == 1).  On a zeroed C with
 *   (1,0) both variants give the same bits.
 * Cells outside [row_start, row_start+N) are never touched. */
static void dd_range(void *p, long lo, long hi)
{
    dd_ctx *c = (dd_ctx *)p;
    float *tmp = c->literal ? NULL : (float *)malloc(sizeof(float) * (size_t)c->h);
    for (long dia = lo; dia < hi; dia++) {
        int k = c->offsets[dia];
        int row_start = c->rf * imax(0, -k);
        int col_start = imax(0, k);
        int N = imin(c->h - row_start, c->rf * (c->w - col_start));
        if (N <= 0) continue;
        float *d_base = c->Cv + (size_t)dia * c->stride + row_start;
        float *acc = c->literal ? d_base : tmp;
        if (!c->literal) for (int n = 0; n < N; n++) acc[n] = 0.f;
        for (int b = 0; b < c->ncols; b++) {
            const float *a = c->A + (size_t)b * c->lda + row_start;
            const float *bb = c->B + (size_t)b * c->ldb + col_start;
            for (int n = 0; n < N; n++) acc[n] += a[n] * bb[n / c->rf];
        }
        if (!c->literal) {
            for (int n = 0; n < N; n++) {
                float s = acc[n];
                if (c->factAB != 1.f) s = c->factAB * s;
                if (c->factC != 0.f) d_base[n] = c->factC * d_base[n] + s;
                else                 d_base[n] = s;
            }
        }
    }
    free(tmp);
}

ORACLE_API int oracle_dd2dia(float *Cvals, const int *offsets, int nd, int h, int w,
                             int stride, int rf, const float *A, int lda,
                             const float *B, int ldb, int ncols,
                             float factAB, float factC, int literal_host, int nthreads)
{
    if (rf <= 0 || stride < h || h % rf != 0) return -1;
    dd_ctx c = { Cvals, offsets, nd, h, w, stride, rf, A, lda, B, ldb, ncols, factAB, factC, literal_host };
    parallel_ranges(dd_range, &c, nd, nthreads);
    return 0;
}

/* ------------------------------------------------------------------------ */
/* reduce_to_col / reduce_to_row                                              */
/* ------------------------------------------------------------------------ */

/* Functor codes: the order of enum reduce_functor, matrix_ops/matrix_ops.hpp:185-196. */
enum { RF_ADD = 0, RF_MEAN, RF_ADD_SQUARED, RF_MAX, RF_ARGMAX, RF_ARGMIN, RF_MIN,
       RF_MULT, RF_LOGADDEXP, RF_ADDEXP };

/* tensor_ops/functors.hpp:520-531 (log1p is log1pf there, functors.hpp uf_log1p) */
static inline float logaddexp_f(float t, float u)
{
    float diff = t - u;
    if (diff > 0) return t + log1pf(expf(-diff));
    else if (diff <= 0) return u + log1pf(expf(diff));
    else return t + u;
}

static inline float rf_init(int rf)
{
    switch (rf) {
    case RF_MAX: case RF_ARGMAX: return -FLT_MAX;            /* functors.hpp:607-610,634-637 */
    case RF_MIN: case RF_ARGMIN: return FLT_MAX;             /* functors.hpp:614-617,641-644 */
    case RF_LOGADDEXP: case RF_ADDEXP: return -INFINITY;     /* functors.hpp:621-624 */
    default: return 0.f;                                     /* functors.hpp:599-602 */
    }
}

/* rv step: fold one raw value into the running result (functors.hpp:453-469,
 * 377-404, 574-594; functor choice per reduce_switch,
 * matrix_ops/matrix_ops_reduce.cu:304-343). */
static inline void rf_rv(int rf, float *r, int *idx, float v, int j)
{
    switch (rf) {
    case RF_ADD: case RF_MEAN: *r = *r + v; break;
    case RF_ADD_SQUARED: *r = *r + v * v; break;
    case RF_MAX: *r = *r > v ? *r : v; break;
    case RF_MIN: *r = *r < v ? *r : v; break;
    case RF_ARGMAX: if (v > *r) { *r = v; *idx = j; } break;
    case RF_ARGMIN: if (v < *r) { *r = v; *idx = j; } break;
    case RF_MULT: *r = *r + logf(v); break;
    case RF_LOGADDEXP: case RF_ADDEXP: *r = logaddexp_f(*r, v); break;
    }
}

typedef struct {
    float *dst; const float *src; long n_contig, n_strided; int over_strided, rf;
    float factNew, factOld;
} red_ctx;

static inline void red_finish(const red_ctx *c, long o, float val, int idx, long n_red)
{
    /* matrix_ops_reduce.cu:277-291 then the post-ops of reduce_switch :308-338 */
    if (c->rf == RF_ARGMAX || c->rf == RF_ARGMIN) { c->dst[o] = (float)idx; return; }
    float r;
    if (c->factOld != 0) r = c->factOld * c->dst[o] + c->factNew * val;
    else                 r = c->factNew * val;
    if (c->rf == RF_MEAN) r = r / (float)n_red;
    if (c->rf == RF_MULT || c->rf == RF_ADDEXP) r = expf(r);
    c->dst[o] = r;
}

static void red_range(void *p, long lo, long hi)
{
    red_ctx *c = (red_ctx *)p;
    if (c->over_strided) {
        /* reduce<1,host>, matrix_ops_reduce.cu:261-268: outputs are the
         * contiguous index; for each strided index in order, fold a whole
         * contiguous line into the outputs.  Split here over output ranges. */
        long n = hi - lo;
        float *val = (float *)malloc(sizeof(float) * n);
        int *idx = (int *)calloc(n, sizeof(int));
        for (long o = 0; o < n; o++) val[o] = rf_init(c->rf);
        for (long j = 0; j < c->n_strided; j++) {
            const float *line = c->src + j * c->n_contig + lo;
            for (long o = 0; o < n; o++) rf_rv(c->rf, &val[o], &idx[o], line[o], (int)j);
        }
        for (long o = 0; o < n; o++) red_finish(c, lo + o, val[o], idx[o], c->n_strided);
        free(val); free(idx);
    } else {
        /* reduce<0,host>, matrix_ops_reduce.cu:254-260: one output per
         * contiguous line, folded sequentially along the line. */
        for (long o = lo; o < hi; o++) {
            float val = rf_init(c->rf); int idx = 0;
            const float *line = c->src + o * c->n_contig;
            for (long j = 0; j < c->n_contig; j++) rf_rv(c->rf, &val, &idx, line[j], (int)j);
            red_finish(c, o, val, idx, c->n_contig);
        }
    }
}

/* src is n_strided lines of n_contig contiguous floats.  over_strided != 0
 * reduces across lines (n_contig outputs: reduce_to_col of a column-major
 * matrix, reduce_to_row of a row-major one, matrix_ops_reduce.cu:348-379);
 * over_strided == 0 reduces along each line (n_strided outputs). */
ORACLE_API int oracle_reduce(float *dst, const float *src, long n_contig, long n_strided,
                             int over_strided, int rf, float factNew, float factOld, int nthreads)
{
    if (rf < RF_ADD || rf > RF_ADDEXP) return -1;
    if (rf == RF_MEAN && !(factNew == 1.f && factOld == 0.f)) return -1; /* matrix_ops_reduce.cu:309-310 */
    red_ctx c = { dst, src, n_contig, n_strided, over_strided, rf, factNew, factOld };
    parallel_ranges(red_range, &c, over_strided ? n_contig : n_strided, nthreads);
    return 0;
}

/* avg_diagonals, host version (matrix_ops/diagonals.cu:23-48): mean of each stored diagonal over the cells
 * inside the matrix, summed sequentially in float; row_fact must be 1 (:28). */
ORACLE_API int oracle_avg_diagonals(float *dst, const float *vals, const int *offsets, int nd, int h, int w, int stride,
                                    int rf)
{
    if (rf != 1) return -1;
    for (int i = 0; i < nd; i++) {
        float sum = 0;
        const int k = offsets[i];
        const int i_start = k < 0 ? -k : 0, j_start = k > 0 ? k : 0;
        const int N = (h - i_start) < (w - j_start) ? (h - i_start) : (w - j_start);
        const float *d = vals + (long)i * stride + i_start;
        for (int j = 0; j < N; j++) sum += *d++;
        dst[i] = sum / N;
    }
    return 0;
}

/* ------------------------------------------------------------------------ */
/* reduce_to_col / reduce_to_row between other element types                  */
/* ------------------------------------------------------------------------ */

/* CUV instantiates the reductions for nine (source S, destination D) pairs
 * (matrix_ops/matrix_ops_reduce.cu:395-413).  The host loop (:217-292) keeps
 * the running value in the SOURCE type (`values` is tensor<unconstV>, :244),
 * starts it at reduce_functor_traits::init_value() (functors.hpp:599-644:
 * 0, or the lowest / highest value of S for max / min and their arg forms),
 * folds with the functors reduce_switch picks (:304-343)
 *    ADD, MEAN     r = bf_plus<D,D,S>(r, x)       = (D)r + (D)x      (functors.hpp:374)
 *    ADD_SQUARED   r = bf_add_square<D,D,S>(r, x) = (D)r + (D)(x*x)  (:392)
 *    MAX, MIN      r = bf_max / bf_min<S,S,S>                        (:401-404)
 *    ARGMAX/ARGMIN reduce_argmax / reduce_argmin<S, index>           (:574-592)
 * (the functor's D result is stored back into the S running value), and ends
 * with  *v = factOld * *v + factNew * r  or  *v = factNew * r  with factors of
 * type S (:277-283), the index for the arg forms (:285-287), and for MEAN a
 * division of v by the line length in D (:312).  The macro below is that loop,
 * sequential, one instance per pair; C's conversions are C++'s. */
#define DEFINE_REDUCE_TYPED(NAME, S, D, S_LOWEST, S_HIGHEST)                                              \
static void NAME(D *dst, const S *src, long n_contig, long n_strided, int over_strided, int rf,          \
                 float factNew_f, float factOld_f)                                                        \
{                                                                                                         \
    const S factNew = (S)factNew_f, factOld = (S)factOld_f;                                               \
    const long n_out = over_strided ? n_contig : n_strided, n_red = over_strided ? n_strided : n_contig;  \
    for (long o = 0; o < n_out; o++) {                                                                    \
        S r = (rf == RF_MAX || rf == RF_ARGMAX) ? (S_LOWEST) : (rf == RF_MIN || rf == RF_ARGMIN) ? (S_HIGHEST) : (S)0; \
        unsigned idx = 0;                                                                                 \
        for (long j = 0; j < n_red; j++) {                                                                \
            const S x = over_strided ? src[j * n_contig + o] : src[o * n_contig + j];                     \
            switch (rf) {                                                                                 \
            case RF_ADD: case RF_MEAN: { const D t = (D)r; r = (S)(D)(t + (D)x); } break;                 \
            case RF_ADD_SQUARED: { const D t = (D)r; r = (S)(D)(t + (D)(x * x)); } break;                 \
            case RF_MAX: r = r > x ? r : x; break;                                                        \
            case RF_MIN: r = r < x ? r : x; break;                                                        \
            case RF_ARGMAX: if (x > r) { r = x; idx = (unsigned)j; } break;                               \
            case RF_ARGMIN: if (x < r) { r = x; idx = (unsigned)j; } break;                               \
            }                                                                                             \
        }                                                                                                 \
        if (rf == RF_ARGMAX || rf == RF_ARGMIN) { dst[o] = (D)idx; continue; }                            \
        if (factOld != 0) dst[o] = factOld * dst[o] + factNew * r;                                        \
        else dst[o] = factNew * r;                                                                        \
        if (rf == RF_MEAN) dst[o] = dst[o] / (D)n_red;                                                    \
    }                                                                                                     \
}

DEFINE_REDUCE_TYPED(red_i32_f32, int, float, INT_MIN, INT_MAX)
DEFINE_REDUCE_TYPED(red_u32_f32, unsigned, float, 0u, UINT_MAX)
DEFINE_REDUCE_TYPED(red_u8_f32, unsigned char, float, 0, 255)
DEFINE_REDUCE_TYPED(red_f32_i32, float, int, -FLT_MAX, FLT_MAX)
DEFINE_REDUCE_TYPED(red_f32_u32, float, unsigned, -FLT_MAX, FLT_MAX)
DEFINE_REDUCE_TYPED(red_f32_u8, float, unsigned char, -FLT_MAX, FLT_MAX)
DEFINE_REDUCE_TYPED(red_u8_u8, unsigned char, unsigned char, 0, 255)
DEFINE_REDUCE_TYPED(red_u8_u32, unsigned char, unsigned, 0, 255)

/* Type codes: 0 float, 1 int, 2 unsigned int, 3 unsigned char.  Returns -1 for a pair CUV does not instantiate,
 * a functor outside ADD/MEAN/ADD_SQUARED/MAX/MIN/ARGMAX/ARGMIN, or MEAN with factors other than (1, 0). */
ORACLE_API int oracle_reduce_typed(void *dst, int dst_type, const void *src, int src_type, long n_contig,
                                   long n_strided, int over_strided, int rf, float factNew, float factOld)
{
    if (!(rf == RF_ADD || rf == RF_MEAN || rf == RF_ADD_SQUARED || rf == RF_MAX || rf == RF_MIN || rf == RF_ARGMAX ||
          rf == RF_ARGMIN)) return -1;
    if (rf == RF_MEAN && !(factNew == 1.f && factOld == 0.f)) return -1;
#define PAIR(ST, DT, FN, S, D) if (src_type == ST && dst_type == DT) { \
        FN((D *)dst, (const S *)src, n_contig, n_strided, over_strided, rf, factNew, factOld); return 0; }
    PAIR(1, 0, red_i32_f32, int, float)
    PAIR(2, 0, red_u32_f32, unsigned, float)
    PAIR(3, 0, red_u8_f32, unsigned char, float)
    PAIR(0, 1, red_f32_i32, float, int)
    PAIR(0, 2, red_f32_u32, float, unsigned)
    PAIR(0, 3, red_f32_u8, float, unsigned char)
    PAIR(3, 3, red_u8_u8, unsigned char, unsigned char)
    PAIR(3, 2, red_u8_u32, unsigned char, unsigned)
#undef PAIR
    return -1;
}

/* ------------------------------------------------------------------------ */
/* RBM step glue (element-wise, column-major [units x batch])                 */
/* ------------------------------------------------------------------------ */

typedef struct { float *act; const float *bias; const float *u; float *sample; long units, ncols; } act_ctx;

/* act <- sigmoid(act + bias[unit]); sample <- act > u ? 1 : 0.
 * matrix_plus_col (matrix_ops/matrix_ops.cu:306-338), SF_SIGM
 * 1/(1+expf(-x)) (tensor_ops/functors.hpp:122) and rnd_binarize's compare
 * (random/random.cu:86-91), in the order examples/rbm/base.py:52-54,93-106
 * applies them.  bias, u and sample may be NULL to skip their stage. */
static void act_range(void *p, long lo, long hi)
{
    act_ctx *c = (act_ctx *)p;
    for (long col = lo; col < hi; col++) {
        float *a = c->act + col * c->units;
        for (long i = 0; i < c->units; i++) {
            float x = a[i];
            if (c->bias) x = x + c->bias[i];
            x = 1.f / (1.f + expf(-x));
            a[i] = x;
            if (c->sample) c->sample[col * c->units + i] = (x > c->u[col * c->units + i]) ? 1.f : 0.f;
        }
    }
}

ORACLE_API void oracle_bias_sigmoid_sample(float *act, const float *bias, const float *u,
                                           float *sample, long units, long ncols, int nthreads)
{
    act_ctx c = { act, bias, u, sample, units, ncols };
    parallel_ranges(act_range, &c, ncols, nthreads);
}

/* ---- gradient step with weight decay -------------------------------------------------------------
 * learn_step_weight_decay (tensor_ops/rprop.cu:331-346): alpha = -learnrate, beta = 1 - learnrate*decay,
 * both formed in float, then W[i] = alpha*dW[i] + beta*W[i]. */
ORACLE_API void oracle_learn_step_weight_decay(float *W, const float *dW, long n, float learnrate, float decay)
{
    const float alpha = -learnrate;
    const float beta = 1.f - learnrate * decay;
    for (long i = 0; i < n; i++)
        W[i] = alpha * dW[i] + beta * W[i];
}

/* learn_step_weight_decay_momentum.  device_formula != 0: the kernel's update (rprop.cu:158-170),
 * m = mw*m - lr*(dW + l2*W); otherwise the host loop as written (rprop.cu:356-367), which has
 * dW - l2*W.  Then W += m and M = m. */
ORACLE_API void oracle_learn_step_weight_decay_momentum(float *W, float *M, const float *dW, long n, float lr,
                                                        float mw, float l2, int device_formula)
{
    for (long i = 0; i < n; i++) {
        float m = M[i];
        if (device_formula)
            m = mw * m - lr * (dW[i] + l2 * W[i]);
        else
            m = mw * m - lr * (dW[i] - l2 * W[i]);
        W[i] += m;
        M[i] = m;
    }
}

/* ---- uniform numbers of the sampling step ---------------------------------------------------------
 * CUV draws the number an activation is binarised against on the device (rnd_binarize, random/random.cu:86-91,
 * 139-156), one generator state per thread, so its stream depends on the launch geometry and no host code
 * reproduces it.  The product path defines the number of element (row, column) of draw `which` in step `step`
 * as word row % 4 of Philox4x32-10 (Salmon, Moraes, Dror, Shaw, "Parallel random numbers: as easy as 1, 2, 3",
 * SC 2011) on counter (row / 4, column, which + 65536 * (column >> 32), step) with key (seed low, seed high),
 * mapped to [0, 1) as (word >> 8) * 2^-24.  This is the published algorithm restated: ten rounds of
 * (hi1 ^ c1 ^ k0, lo1, hi0 ^ c3 ^ k1, lo0) with (hi0, lo0) = 0xD2511F53 * c0, (hi1, lo1) = 0xCD9E8D57 * c2, the key
 * raised by (0x9E3779B9, 0xBB67AE85) between rounds.  Pinned by the known-answer vectors of the generator's
 * authors in tests/test_oracle_golden.py. */
ORACLE_API void oracle_philox4x32_10(const unsigned *ctr, const unsigned *key, unsigned *out)
{
    unsigned c0 = ctr[0], c1 = ctr[1], c2 = ctr[2], c3 = ctr[3], k0 = key[0], k1 = key[1];
    for (int r = 0; r < 10; r++) {
        const unsigned long long p0 = 0xD2511F53ull * c0, p1 = 0xCD9E8D57ull * c2;
        const unsigned n0 = (unsigned)(p1 >> 32) ^ c1 ^ k0, n1 = (unsigned)p1;
        const unsigned n2 = (unsigned)(p0 >> 32) ^ c3 ^ k1, n3 = (unsigned)p0;
        c0 = n0; c1 = n1; c2 = n2; c3 = n3;
        k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
    }
    out[0] = c0; out[1] = c1; out[2] = c2; out[3] = c3;
}

ORACLE_API void oracle_uniform(float *dst, long ld, long rows, long ncols, unsigned long long seed,
                               unsigned long long step, long long col0, int which)
{
    const unsigned key[2] = {(unsigned)(seed & 0xffffffffull), (unsigned)(seed >> 32)};
    for (long c = 0; c < ncols; c++) {
        const long long gcol = col0 + c;
        for (long q = 0; 4 * q < rows; q++) {
            const unsigned ctr[4] = {(unsigned)q, (unsigned)gcol, (unsigned)which + 65536u * (unsigned)(gcol >> 32),
                                     (unsigned)step};
            unsigned w[4];
            oracle_philox4x32_10(ctr, key, w);
            for (int e = 0; e < 4 && 4 * q + e < rows; e++)
                dst[c * ld + 4 * q + e] = (float)(w[e] >> 8) * (1.f / 16777216.f);
        }
    }
}
