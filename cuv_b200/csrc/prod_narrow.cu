// prod with a banded DIA operand (row_fact 1) in the memory-bound regime: few diagonals and/or few
// batch columns (the classical DIA use: a penta-diagonal operator times a handful of vectors).
//
// Here every byte of A, B and C should cross HBM exactly once and nothing else matters.  A thread
// owns 4 consecutive output rows and walks the band 16 diagonals at a time.  For 4 batch columns at
// once it loads the 19 consecutive B rows those 4 x 16 cells touch as six aligned 128-bit loads per
// column into registers (a sliding window: cell (row j, diagonal k) reads window entry rem + j + k,
// a compile-time index because the band's alignment `rem` is a template parameter), and the
// coefficients as one aligned 128-bit load per diagonal (two for the transposed product, whose
// diagonal is read at a shifting row).  Neighbouring threads overlap in the B rows they load; that
// overlap is served by L1, HBM sees each row once.  The block loops over the column groups itself,
// so its slice of A is re-read from L1/L2, not from HBM.  No shared memory, no barriers.
// Accumulation per output is in diagonal storage order; EXACT uses a separate multiply and add and
// reproduces CUV's host loop (matrix_ops/spmv.cu:161-198) bit for bit.
#include <cuda.h>

#include "cuvdia_internal.cuh"

namespace cuvdia {

namespace pn {
constexpr int THREADS = 128;
constexpr int KD = 16;       // diagonals per pass
constexpr int CB = 4;        // batch columns per pass
constexpr int NW = 6;        // 128-bit loads per column: 24 window entries >= 3 + 19
}

struct NarrowParams {
    int h, w, nd, lo, S;
    int ldb, ldc, ncols;
    float fa, fc;
    const float* A; const float* B; float* C;
};

// One pass: 16 diagonals (kb .. kb+15) x 4 rows x CB columns accumulated into acc.
// L = lo mod 4 (non-negative).  'n': window entry of cell (j,k) is L + j + k, window starts at row
// i0 + lo + kb - L.  't': cell (j,k) reads matrix row i0 - lo - kb + j - k; the window starts 15 + RT rows
// below i0 - lo - kb with RT = (1 - lo) mod 4, entry 15 + RT + j - k; the coefficients of diagonal k start at
// offset (RA - k) mod 4 of an aligned 8-vector, RA = (-lo) mod 4.
// FAST: the caller has checked that every load of the pass is inside the operands and every cell inside the
// matrix, so the pass is straight-line code: 6*CB + 16 (or 32) vector loads issued back to back, then the
// multiply-adds.  Otherwise every load and cell is guarded.
template <bool TRANS, bool EXACT, int L, bool FAST>
__device__ __forceinline__ void narrow_pass(const NarrowParams& P, float (&acc)[pn::CB][4], int i0, int c0, int kb) {
    using namespace pn;
    constexpr int RA = (4 - L) % 4;
    constexpr int RT = (RA + 1) % 4;
    const int rows_b = TRANS ? P.h : P.w;
    const int ws = TRANS ? (i0 - P.lo - kb - 15 - RT) : (i0 + P.lo + kb - L);      // first row of the window, a multiple of 4
    float wv[CB][4 * NW];
#pragma unroll
    for (int c = 0; c < CB; c++) {
        const bool col_ok = FAST || c0 + c < P.ncols;
        const float* bp = P.B + (size_t)(col_ok ? c0 + c : 0) * P.ldb;
#pragma unroll
        for (int v = 0; v < NW; v++) {
            const int r = ws + 4 * v;
            float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
            if (FAST || (col_ok && r >= 0 && r + 4 <= rows_b)) {
                x = __ldg(reinterpret_cast<const float4*>(bp + r));
            } else if (col_ok && r + 3 >= 0 && r < rows_b) {
                if (r >= 0) x.x = __ldg(bp + r);
                if (r + 1 >= 0 && r + 1 < rows_b) x.y = __ldg(bp + r + 1);
                if (r + 2 >= 0 && r + 2 < rows_b) x.z = __ldg(bp + r + 2);
                if (r + 3 >= 0 && r + 3 < rows_b) x.w = __ldg(bp + r + 3);
            }
            wv[c][4 * v] = x.x; wv[c][4 * v + 1] = x.y; wv[c][4 * v + 2] = x.z; wv[c][4 * v + 3] = x.w;
        }
    }
    float a[KD][4];
#pragma unroll
    for (int k = 0; k < KD; k++) {
        const float* Ak = P.A + (size_t)(kb + k) * P.S;
        if (!TRANS) {
            if (FAST) {
                const float4 t = __ldg(reinterpret_cast<const float4*>(Ak + i0));
                a[k][0] = t.x; a[k][1] = t.y; a[k][2] = t.z; a[k][3] = t.w;
            } else {
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const int jb = i0 + j + P.lo + kb + k;                    // matrix column of the cell
                    const bool ok = kb + k < P.nd && i0 + j < P.h && jb >= 0 && jb < P.w;
                    a[k][j] = ok ? __ldg(Ak + i0 + j) : 0.f;
                }
            }
        } else {
            const int off = ((RA - k) % 4 + 4) % 4;
            const int i = i0 - P.lo - kb - k;                                  // matrix row of cell (0, k)
            if (FAST) {
                const float4 t0 = __ldg(reinterpret_cast<const float4*>(Ak + (i - off)));
                const float4 t1 = __ldg(reinterpret_cast<const float4*>(Ak + (i - off) + 4));
                const float av[8] = {t0.x, t0.y, t0.z, t0.w, t1.x, t1.y, t1.z, t1.w};
#pragma unroll
                for (int j = 0; j < 4; j++) a[k][j] = av[off + j];
            } else {
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const int ii = i + j;
                    const bool ok = kb + k < P.nd && i0 + j < P.w && ii >= 0 && ii < P.h;
                    a[k][j] = ok ? __ldg(Ak + ii) : 0.f;
                }
            }
        }
    }
#pragma unroll
    for (int k = 0; k < KD; k++)
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const float t = (P.fa != 1.f) ? __fmul_rn(P.fa, a[k][j]) : a[k][j];
#pragma unroll
            for (int c = 0; c < CB; c++) {
                const float x = TRANS ? wv[c][15 + RT + j - k] : wv[c][L + j + k];
                acc[c][j] = EXACT ? __fadd_rn(acc[c][j], __fmul_rn(t, x)) : fmaf(t, x, acc[c][j]);
            }
        }
}

template <bool TRANS, bool EXACT, int L>
__global__ void __launch_bounds__(pn::THREADS)
prod_narrow_kernel(const NarrowParams P) {
    using namespace pn;
    constexpr int RT = ((4 - L) % 4 + 1) % 4;
    const int rows_out = TRANS ? P.w : P.h;
    const int rows_b = TRANS ? P.h : P.w;
    const int i0 = 4 * (blockIdx.x * THREADS + threadIdx.x);
    if (i0 >= rows_out) return;
    const bool full_rows = i0 + 4 <= rows_out;
    const bool vec_c = (P.ldc & 3) == 0 && (reinterpret_cast<uintptr_t>(P.C) & 15) == 0;

    for (int c0 = 0; c0 < P.ncols; c0 += CB) {
        float acc[CB][4];
#pragma unroll
        for (int c = 0; c < CB; c++)
#pragma unroll
            for (int j = 0; j < 4; j++) {
                acc[c][j] = 0.f;
                if (P.fc != 0.f && c0 + c < P.ncols && i0 + j < rows_out)
                    acc[c][j] = __fmul_rn(P.C[(size_t)(c0 + c) * P.ldc + i0 + j], P.fc);
            }
        for (int kb = 0; kb < P.nd; kb += KD) {
            // the whole window (24 rows from ws) inside the operand, every diagonal of the pass stored, all four
            // rows and all CB columns present: then nothing needs a guard
            const int ws = TRANS ? (i0 - P.lo - kb - 15 - RT) : (i0 + P.lo + kb - L);
            const bool fast = full_rows && c0 + CB <= P.ncols && kb + KD <= P.nd && ws >= 0 && ws + 4 * NW <= rows_b;
            if (fast) narrow_pass<TRANS, EXACT, L, true>(P, acc, i0, c0, kb);
            else narrow_pass<TRANS, EXACT, L, false>(P, acc, i0, c0, kb);
        }
#pragma unroll
        for (int c = 0; c < CB; c++) {
            if (c0 + c >= P.ncols) continue;
            float* cp = P.C + (size_t)(c0 + c) * P.ldc + i0;
            if (full_rows && vec_c) {
                *reinterpret_cast<float4*>(cp) = make_float4(acc[c][0], acc[c][1], acc[c][2], acc[c][3]);
            } else {
#pragma unroll
                for (int j = 0; j < 4; j++)
                    if (i0 + j < rows_out) cp[j] = acc[c][j];
            }
        }
    }
}

// ------------------------------------------------------------------------------------------------
// Streaming variant for bands of at most 16 diagonals: the same arithmetic, but A and B reach the SM
// through TMA (cp.async.bulk.tensor, no multicast) instead of through per-thread loads.  An SM can
// keep only so many L1 misses in flight, which caps prod_narrow_kernel at about a third of the HBM
// bandwidth; the copy engine has no such limit.  A block owns 512 output rows: its slice of the
// band (16 x 544 floats) and the B window of up to 32 batch columns (544 rows each) are fetched by
// eight tile loads onto one mbarrier (bounded wait), two blocks share an SM so one computes while
// the other's loads are in flight.  The coefficients of a thread's 4 rows stay in registers for all
// column groups.  Tiles are 136 rows tall (4 x 34: TMA boxes are limited to 256 rows); a window row
// r lives at [r / 136][column][r % 136].
// ------------------------------------------------------------------------------------------------
namespace ps {
constexpr int THREADS = 128;
constexpr int TR = 4 * THREADS;       // output rows per block
constexpr int BOXR = 136;             // rows per TMA box
constexpr int NBOX = 4;               // boxes per window: 544 rows >= 512 + 24 + 3
constexpr int NC = 32;                // batch columns per round
constexpr int A_FLOATS = NBOX * pn::KD * BOXR;
constexpr int B_FLOATS = NBOX * NC * BOXR;
constexpr size_t SMEM = sizeof(float) * (A_FLOATS + B_FLOATS) + 64;
constexpr unsigned SPIN_LIMIT = 1u << 26;
}

struct StreamParams {
    int h, w, nd, lo, ldc, ncols;
    float fa, fc;
    float* C;
    int* status;
};

__device__ __forceinline__ unsigned s_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }

// element (window row r, plane y) of a buffer made of NBOX boxes of [planes][BOXR]
__device__ __forceinline__ int box_index(int r, int y, int planes) {
    const int b = (r >= ps::BOXR) + (r >= 2 * ps::BOXR) + (r >= 3 * ps::BOXR);
    return (b * planes + y) * ps::BOXR + (r - b * ps::BOXR);
}

template <bool TRANS, bool EXACT, int L>
__global__ void __launch_bounds__(ps::THREADS, 2)
prod_stream_kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB,
                   const StreamParams P) {
    using namespace ps;
    constexpr int KD = pn::KD, CB = pn::CB, NW = pn::NW;
    constexpr int RA = (4 - L) % 4;
    constexpr int RT = (RA + 1) % 4;
    extern __shared__ __align__(1024) float sm[];
    float* const As = sm;                       // [NBOX][KD][BOXR]
    float* const Bs = sm + A_FLOATS;            // [NBOX][NC][BOXR]
    unsigned long long* const bar = reinterpret_cast<unsigned long long*>(sm + A_FLOATS + B_FLOATS);
    const int tid = threadIdx.x;
    const int o0 = blockIdx.x * TR;             // first output row of the block
    const int rows_out = TRANS ? P.w : P.h;
    const int rows_b = TRANS ? P.h : P.w;
    // first matrix row of the B window (multiple of 4) and of the A window
    const int wsB = TRANS ? (o0 - P.lo - (KD - 1) - RT) : (o0 + P.lo - L);
    const int wsA = TRANS ? wsB : o0;
    if (tid == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(s_u32(bar)));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    const int i0 = o0 + 4 * tid;                // this thread's 4 output rows
    // block-uniform: every cell the block touches lies inside the matrix and every output row exists
    const int cell0 = TRANS ? (o0 - P.lo - (KD - 1)) : (o0 + P.lo);
    const bool interior = P.nd == KD && o0 + TR <= rows_out && cell0 >= 0 && cell0 + TR - 1 + (KD - 1) < rows_b;
    float a[KD][4];
    unsigned phase = 0;
    for (int cbase = 0; cbase < P.ncols; cbase += NC) {
        if (tid == 0) {
            const unsigned nbytes = sizeof(float) * ((cbase == 0 ? A_FLOATS : 0) + B_FLOATS);
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(s_u32(bar)), "r"(nbytes) : "memory");
#pragma unroll
            for (int b = 0; b < NBOX; b++) {
                if (cbase == 0)
                    asm volatile(
                        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                        ::"r"(s_u32(As + b * KD * BOXR)), "l"(&mapA), "r"(wsA + b * BOXR), "r"(0), "r"(s_u32(bar)) : "memory");
                asm volatile(
                    "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                    ::"r"(s_u32(Bs + b * NC * BOXR)), "l"(&mapB), "r"(wsB + b * BOXR), "r"(cbase), "r"(s_u32(bar)) : "memory");
            }
        }
        bool done = false;
        for (unsigned it = 0; it < SPIN_LIMIT && !done; it++) {
            unsigned d;
            asm volatile(
                "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                : "=r"(d) : "r"(s_u32(bar)), "r"(phase) : "memory");
            done = d != 0;
        }
        if (!done) { if (P.status) *P.status = 3; return; }
        phase ^= 1;
        if (cbase == 0) {
            // coefficients of this thread's 4 rows, kept in registers for every column group
#pragma unroll
            for (int k = 0; k < KD; k++) {
                if (!TRANS) {
                    const float4 t = *reinterpret_cast<const float4*>(As + box_index(4 * tid, k, KD));
                    a[k][0] = t.x; a[k][1] = t.y; a[k][2] = t.z; a[k][3] = t.w;
                } else {
                    // cell (j,k) reads matrix row i0 - lo - k + j = wsA + (KD-1) + RT + 4*tid - k + j
                    const int off = ((RA - k) % 4 + 4) % 4;
                    const int r = (KD - 1) + RT + 4 * tid - k - off;       // aligned window row
                    const float4 t0 = *reinterpret_cast<const float4*>(As + box_index(r, k, KD));
                    const float4 t1 = *reinterpret_cast<const float4*>(As + box_index(r + 4, k, KD));
                    const float av[8] = {t0.x, t0.y, t0.z, t0.w, t1.x, t1.y, t1.z, t1.w};
#pragma unroll
                    for (int j = 0; j < 4; j++) a[k][j] = av[off + j];
                }
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    if (!interior) {
                        // cells outside the matrix (their storage may hold anything) count as zero
                        const int x = TRANS ? (i0 + j - P.lo - k) : (i0 + j + P.lo + k);   // matrix row ('t') or column ('n')
                        const bool ok = k < P.nd && i0 + j < rows_out && x >= 0 && x < rows_b;
                        if (!ok) a[k][j] = 0.f;
                    }
                    if (P.fa != 1.f) a[k][j] = __fmul_rn(P.fa, a[k][j]);
                }
            }
        }
        const int ncb = min(NC, P.ncols - cbase);
        for (int c0 = 0; c0 < ncb; c0 += CB) {
            float acc[CB][4];
            float wv[CB][4 * NW];
#pragma unroll
            for (int c = 0; c < CB; c++) {
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    acc[c][j] = 0.f;
                    if (P.fc != 0.f && c0 + c < ncb && i0 + j < rows_out)
                        acc[c][j] = __fmul_rn(P.C[(size_t)(cbase + c0 + c) * P.ldc + i0 + j], P.fc);
                }
#pragma unroll
                for (int v = 0; v < NW; v++) {
                    const float4 x = *reinterpret_cast<const float4*>(Bs + box_index(4 * tid + 4 * v, min(c0 + c, NC - 1), NC));
                    wv[c][4 * v] = x.x; wv[c][4 * v + 1] = x.y; wv[c][4 * v + 2] = x.z; wv[c][4 * v + 3] = x.w;
                }
            }
#pragma unroll
            for (int k = 0; k < KD; k++)
#pragma unroll
                for (int j = 0; j < 4; j++)
#pragma unroll
                    for (int c = 0; c < CB; c++) {
                        const float x = TRANS ? wv[c][(KD - 1) + RT + j - k] : wv[c][L + j + k];
                        acc[c][j] = EXACT ? __fadd_rn(acc[c][j], __fmul_rn(a[k][j], x)) : fmaf(a[k][j], x, acc[c][j]);
                    }
            const bool vec_c = (P.ldc & 3) == 0 && (reinterpret_cast<uintptr_t>(P.C) & 15) == 0 && i0 + 4 <= rows_out;
#pragma unroll
            for (int c = 0; c < CB; c++) {
                if (c0 + c >= ncb) continue;
                float* cp = P.C + (size_t)(cbase + c0 + c) * P.ldc + i0;
                if (vec_c) *reinterpret_cast<float4*>(cp) = make_float4(acc[c][0], acc[c][1], acc[c][2], acc[c][3]);
                else {
#pragma unroll
                    for (int j = 0; j < 4; j++)
                        if (i0 + j < rows_out) cp[j] = acc[c][j];
                }
            }
        }
        __syncthreads();          // all threads are done with the B window before the next round overwrites it
    }
}

static inline bool al16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// Banded, row_fact 1, 16-byte aligned operands, and little enough work per output row that HBM
// traffic, not arithmetic, decides the time.
bool prod_narrow_applicable(const cuvdia_plan* p, const float* A, const float* B, int ldb, int ncols) {
    if (!(p->is_band && p->rf == 1 && al16(A) && al16(B) && p->stride % 4 == 0 && ldb % 4 == 0)) return false;
    return (long long)p->nd * ncols <= 2048 && (ncols < 64 || p->nd < 24);
}

template <bool TRANS, bool EXACT>
static int launch_narrow_t(const cuvdia_plan* p, const NarrowParams& P, cudaStream_t st) {
    const int rows_out = TRANS ? p->w : p->h;
    const int threads_needed = (rows_out + 3) / 4;
    const int blocks = (threads_needed + pn::THREADS - 1) / pn::THREADS;
    const int L = ((p->band_lo % 4) + 4) % 4;
    switch (L) {
        case 0: prod_narrow_kernel<TRANS, EXACT, 0><<<blocks, pn::THREADS, 0, st>>>(P); break;
        case 1: prod_narrow_kernel<TRANS, EXACT, 1><<<blocks, pn::THREADS, 0, st>>>(P); break;
        case 2: prod_narrow_kernel<TRANS, EXACT, 2><<<blocks, pn::THREADS, 0, st>>>(P); break;
        default: prod_narrow_kernel<TRANS, EXACT, 3><<<blocks, pn::THREADS, 0, st>>>(P); break;
    }
    count_launch();
    return check_launch("prod_narrow_kernel");
}

int make_map_2d(CUtensorMap* m, const float* base, long long dim0, long long dim1, long long pitch, int box0, int box1);

template <bool TRANS, bool EXACT>
static int launch_stream_t(const cuvdia_plan* p, const float* A, const float* B, int ldb, float* C, int ldc, int ncols,
                           float fa, float fc, cudaStream_t st) {
    using namespace ps;
    CUtensorMap mapA, mapB;
    int rc = make_map_2d(&mapA, A, p->h, p->nd, p->stride, BOXR, pn::KD);
    if (rc) return rc;
    rc = make_map_2d(&mapB, B, TRANS ? p->h : p->w, ncols, ldb, BOXR, NC);
    if (rc) return rc;
    StreamParams P;
    P.h = p->h; P.w = p->w; P.nd = p->nd; P.lo = p->band_lo; P.ldc = ldc; P.ncols = ncols;
    P.fa = fa; P.fc = fc; P.C = C; P.status = p->d_status;
    const int rows_out = TRANS ? p->w : p->h;
    const int blocks = (rows_out + TR - 1) / TR;
    const int L = ((p->band_lo % 4) + 4) % 4;
#define GO(LV)                                                                                          \
    do {                                                                                                \
        static bool attr[64] = {false};                                                                 \
        rc = allow_dynamic_smem(prod_stream_kernel<TRANS, EXACT, LV>, SMEM, attr);                      \
        if (rc) return rc;                                                                              \
        prod_stream_kernel<TRANS, EXACT, LV><<<blocks, THREADS, SMEM, st>>>(mapA, mapB, P);             \
    } while (0)
    switch (L) { case 0: GO(0); break; case 1: GO(1); break; case 2: GO(2); break; default: GO(3); break; }
#undef GO
    count_launch();
    return check_launch("prod_stream_kernel");
}

// The streaming variant needs the whole band in one pass and enough rows to fill the GPU.
bool prod_narrow_streams(const cuvdia_plan* p, bool trans) {
    return p->nd <= pn::KD && (trans ? p->w : p->h) >= 64 * ps::TR && tma_available();
}

int launch_prod_narrow(const cuvdia_plan* p, const float* A, const float* B, int ldb, float* C, int ldc, int ncols,
                       bool trans, float fa, float fc, int mode, cudaStream_t st) {
    if (prod_narrow_streams(p, trans)) {
        const bool ex = mode == CUVDIA_MODE_EXACT;
        if (trans) return ex ? launch_stream_t<true, true>(p, A, B, ldb, C, ldc, ncols, fa, fc, st)
                             : launch_stream_t<true, false>(p, A, B, ldb, C, ldc, ncols, fa, fc, st);
        return ex ? launch_stream_t<false, true>(p, A, B, ldb, C, ldc, ncols, fa, fc, st)
                  : launch_stream_t<false, false>(p, A, B, ldb, C, ldc, ncols, fa, fc, st);
    }
    NarrowParams P;
    P.h = p->h; P.w = p->w; P.nd = p->nd; P.lo = p->band_lo; P.S = p->stride;
    P.ldb = ldb; P.ldc = ldc; P.ncols = ncols; P.fa = fa; P.fc = fc; P.A = A; P.B = B; P.C = C;
    const bool exact = mode == CUVDIA_MODE_EXACT;
    if (trans) return exact ? launch_narrow_t<true, true>(p, P, st) : launch_narrow_t<true, false>(p, P, st);
    return exact ? launch_narrow_t<false, true>(p, P, st) : launch_narrow_t<false, false>(p, P, st);
}

}  // namespace cuvdia
