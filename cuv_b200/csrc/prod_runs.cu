// prod with a DIA operand whose stored diagonals come in runs of consecutive numbers (row_fact 1):
// the pattern of a convolution written as a sparse matrix - a filter row is a run of `fs` diagonals,
// the next filter row starts one image line further (basics/filter_factory.hpp:43-76; CUV's own
// speed fixture uses off = i*px + j, src/tests/spmv_speed.cpp:96-104).  Neither a band nor a
// scattered set: the span of the offsets is large, but inside a run neighbouring diagonals share
// all but one of the dense operand's rows.
//
// The plan cuts the offset list, in storage order, into passes of up to 8 consecutive diagonals.
// A block owns 256 output rows and up to 16 batch columns and walks the passes in order.  A matrix
// of this kind has few rows, hence few warps, and every pass needs another slice of the coefficients
// (used once, from HBM) and another window of the dense operand (from L2): per-thread loads cannot
// keep enough of them in flight.  So one producer thread streams both through a four-stage ring in
// shared memory with TMA tile loads (cp.async.bulk.tensor, no multicast; rows or diagonals outside
// the operands arrive as zeros) and full/empty mbarriers with bounded waits, two blocks per SM, and
// asks for the coefficient tiles a dozen passes ahead to be brought into L2 (tensor prefetch), while
// 128 consumer threads compute: a thread owns 4 rows and 8 of the columns, reads the 8 x 4
// coefficients of the pass and, per column, the 11 dense rows its 4 x 8 cells touch as three or four
// aligned 128-bit shared loads into a register window (cell (row j, diagonal k) reads entry L + j + k, L = alignment of the run's first
// offset, a template parameter so that the index is a compile-time constant), then issues 32
// multiply-adds.  Passes that touch the border of the matrix, or are shorter than 8, zero the
// coefficients of cells outside the matrix (the dense rows they would read are outside too and
// arrive as zeros) and skip the diagonals that are not part of the pass.
// Accumulation per output is in diagonal storage order; EXACT uses a separate multiply and add and
// reproduces CUV's host loop (matrix_ops/spmv.cu:161-198) bit for bit, repeated offsets included.
#include <cuda.h>

#include "cuvdia_internal.cuh"

namespace cuvdia {

int make_map_2d(CUtensorMap* m, const float* base, long long dim0, long long dim1, long long pitch, int box0, int box1);

namespace pr {
constexpr int ROWTHREADS = 64;              // threads along the rows; each owns 4 consecutive rows
constexpr int CONSUMERS = 2 * ROWTHREADS;   // two halves of the block's columns
constexpr int THREADS = CONSUMERS + 32;     // four consumer warps and the producer's warp
constexpr int TR = 4 * ROWTHREADS;          // output rows per block
constexpr int KD = 8;                       // diagonals per pass
constexpr int CG = 16;                      // batch columns per block
constexpr int CT = CG / 2;                  // batch columns per thread
constexpr int NW = 4;                       // 128-bit loads per column: 16 window entries >= 3 + 4 + 7
constexpr int BOXR = 136;                   // rows per TMA box of a window of TR + 16 rows (two boxes)
constexpr int NS = 4;                       // ring stages
constexpr int A_FLOATS = 2 * KD * BOXR;
constexpr int B_FLOATS = 2 * CG * BOXR;
constexpr int STAGE_FLOATS = A_FLOATS + B_FLOATS;
constexpr size_t SMEM = sizeof(float) * NS * STAGE_FLOATS + 2 * NS * sizeof(unsigned long long);
constexpr int AHEAD = 12;                   // passes between the L2 prefetch of a coefficient tile and its load
constexpr unsigned SPIN_LIMIT = 1u << 26;
template <bool TRANS> __host__ __device__ constexpr int abox() { return TRANS ? BOXR : TR / 2; }
template <bool TRANS> __host__ __device__ constexpr unsigned stage_bytes() {
    return sizeof(float) * (2 * KD * abox<TRANS>() + B_FLOATS);
}
}

struct RunsParams {
    int h, w, ldc, ncols, npass;
    int off_min, off_max;
    float fa, fc;
    float* C;
    const int4* passes;      // (first slot, first offset, diagonals, unused) per pass
    int* status;
};

__device__ __forceinline__ unsigned r_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }

// A pass descriptor, read-only path.  Volatile so that the load stays where it is written - at the top of an
// iteration, a whole pass before its value is needed - instead of sinking to its first use.
__device__ __forceinline__ int4 ld_desc(const int4* p) {
    int4 v;
    asm volatile("ld.global.nc.v4.s32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

// bounded wait on an mbarrier phase; false if it gave up
__device__ __forceinline__ bool r_wait(unsigned long long* bar, unsigned parity) {
    for (unsigned it = 0; it < pr::SPIN_LIMIT; it++) {
        unsigned d;
        asm volatile(
            "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(d) : "r"(r_u32(bar)), "r"(parity) : "memory");
        if (d) return true;
    }
    return false;
}

// One pass out of a ring stage.
// 'n': the stage's window starts at dense row o0 + lo - L; a thread's entries start 4*tid further; cell (j,k)
//      reads entry L + j + k.  Coefficients: rows o0.. in two boxes of 128.
// 't': cell (j,k) reads matrix row i0 + j - lo - k; the window starts 7 + RT rows below o0 - lo with
//      RT = (1 - lo) mod 4, entry 7 + RT + j - k; the coefficients share the window's rows, those of diagonal k
//      start at offset (RA - k) mod 4 of an aligned 8-vector, RA = (-lo) mod 4.
template <bool TRANS, bool EXACT, int L, bool INTERIOR>
__device__ __forceinline__ void runs_pass(const float* __restrict__ As, const float* __restrict__ Bs,
                                          float (&acc)[pr::CT][4], const int (&hoff)[pr::NW], int tid, int nc,
                                          const RunsParams& P, int i0, int lo, int cnt) {
    using namespace pr;
    constexpr int RA = (4 - L) % 4;
    constexpr int RT = (RA + 1) % 4;
    constexpr int AB = abox<TRANS>();
    float a[KD][4];
#pragma unroll
    for (int k = 0; k < KD; k++) {
        if (!TRANS) {
            const int r = 4 * tid, b = r >= AB ? 1 : 0;
            const float4 t = *reinterpret_cast<const float4*>(As + (b * KD + k) * AB + (r - b * AB));
            a[k][0] = t.x; a[k][1] = t.y; a[k][2] = t.z; a[k][3] = t.w;
        } else {
            const int off = ((RA - k) % 4 + 4) % 4;
            const int r0 = 4 * tid + (KD - 1) + RT - k - off, r1 = r0 + 4;      // aligned window rows
            const int b0 = r0 >= AB ? 1 : 0, b1 = r1 >= AB ? 1 : 0;
            const float4 t0 = *reinterpret_cast<const float4*>(As + (b0 * KD + k) * AB + (r0 - b0 * AB));
            const float4 t1 = *reinterpret_cast<const float4*>(As + (b1 * KD + k) * AB + (r1 - b1 * AB));
            const float av[8] = {t0.x, t0.y, t0.z, t0.w, t1.x, t1.y, t1.z, t1.w};
#pragma unroll
            for (int j = 0; j < 4; j++) a[k][j] = av[off + j];
        }
#pragma unroll
        for (int j = 0; j < 4; j++) {
            if (!INTERIOR) {
                // cells outside the matrix (their storage may hold anything) count as zero
                const int x = TRANS ? (i0 + j - lo - k) : (i0 + j + lo + k);      // matrix row ('t') or column ('n')
                const bool ok = k < cnt && i0 + j < (TRANS ? P.w : P.h) && x >= 0 && x < (TRANS ? P.h : P.w);
                if (!ok) a[k][j] = 0.f;
            }
            if (P.fa != 1.f) a[k][j] = __fmul_rn(P.fa, a[k][j]);
        }
    }
    // entries the cells use: 'n' L .. L+10, 't' RT .. RT+10; the last 128-bit load is needed only beyond 12
    constexpr int NWL = ((TRANS ? RT : L) + 11 + 3) / 4;
    // Two columns at a time: eight independent accumulation chains.  A pair is computed if its first column
    // exists; a second column past the batch reads the zeros TMA wrote there and its sums are never stored.
#pragma unroll
    for (int c = 0; c < CT; c += 2) {
        if (c < nc) {
            float wv[2][4 * NW];
#pragma unroll
            for (int cc = 0; cc < 2; cc++)
#pragma unroll
                for (int v = 0; v < NWL; v++) {
                    const float4 x = *reinterpret_cast<const float4*>(Bs + hoff[v] + (c + cc) * BOXR);
                    wv[cc][4 * v] = x.x; wv[cc][4 * v + 1] = x.y; wv[cc][4 * v + 2] = x.z; wv[cc][4 * v + 3] = x.w;
                }
#pragma unroll
            for (int k = 0; k < KD; k++) {
                if (INTERIOR || k < cnt) {
#pragma unroll
                    for (int j = 0; j < 4; j++) {
#pragma unroll
                        for (int cc = 0; cc < 2; cc++) {
                            const float x = wv[cc][TRANS ? (KD - 1) + RT + j - k : L + j + k];
                            acc[c + cc][j] = EXACT ? __fadd_rn(acc[c + cc][j], __fmul_rn(a[k][j], x))
                                                   : fmaf(a[k][j], x, acc[c + cc][j]);
                        }
                    }
                }
            }
        }
    }
}

template <bool TRANS, bool EXACT>
__global__ void __launch_bounds__(pr::THREADS, 2)
prod_runs_kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB,
                 const RunsParams P) {
    using namespace pr;
    extern __shared__ __align__(1024) float sm[];
    unsigned long long* const full = reinterpret_cast<unsigned long long*>(sm + NS * STAGE_FLOATS);
    unsigned long long* const empty = full + NS;
    const int tid = threadIdx.x;
    const int rows_out = TRANS ? P.w : P.h;
    const int ngroups = (P.ncols + CG - 1) / CG;
    const int cgi = blockIdx.x % ngroups;                 // column groups of one row block are neighbours in launch
    const int rb = blockIdx.x / ngroups;                  // order, so they find its coefficients in L2
    const int c0 = cgi * CG;
    const int o0 = rb * TR;
    if (tid == 0) {
        for (int s = 0; s < NS; s++) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(r_u32(full + s)));
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 4;" ::"r"(r_u32(empty + s)));     // one arrival per consumer warp
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    // rows of this block that no stored diagonal reaches only get scaled
    const bool reachable = TRANS ? (o0 + TR - 1 >= P.off_min && o0 <= P.h - 1 + P.off_max)
                                 : (o0 + TR - 1 + P.off_max >= 0 && o0 + P.off_min < P.w);
    // a pass none of whose cells lies in the block's rows is skipped by producer and consumers alike
    auto touches = [&](int lo, int cnt) {
        return TRANS ? (o0 + TR - 1 - lo >= 0 && o0 - lo - (cnt - 1) < P.h)
                     : (o0 + TR - 1 + lo + cnt - 1 >= 0 && o0 + lo < P.w);
    };

    if (tid >= CONSUMERS) {
        // ---- producer: one thread feeds the ring ----
        if (tid != CONSUMERS || !reachable) return;
        // The coefficients come from HBM, and four stages do not cover that latency: ask for the tiles of a
        // later pass to be brought into L2 now, so that the ring's loads find them there.
        auto prefetch_A = [&](int p) {
            const int4 e = __ldg(P.passes + p);
            if (!touches(e.y, e.z)) return;
            const int Lp = ((e.y % 4) + 4) % 4;
            const int RTp = (((4 - Lp) % 4) + 1) % 4;
            const int x0 = TRANS ? (o0 - e.y - (KD - 1) - RTp) : o0;
#pragma unroll
            for (int b = 0; b < 2; b++)
                asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];"
                             ::"l"(&mapA), "r"(x0 + b * abox<TRANS>()), "r"(e.x) : "memory");
        };
        for (int p = NS; p < min(AHEAD, P.npass); p++) prefetch_A(p);
        int n = 0;
        for (int p = 0; p < P.npass; p++) {
            const int4 d = __ldg(P.passes + p);
            const int slot0 = d.x, lo = d.y, cnt = d.z;
            if (p + AHEAD < P.npass) prefetch_A(p + AHEAD);
            if (!touches(lo, cnt)) continue;
            const int s = n % NS;
            if (n >= NS && !r_wait(empty + s, ((n / NS) - 1) & 1)) { if (P.status) *P.status = 5; break; }
            float* const As = sm + s * STAGE_FLOATS;
            float* const Bs = As + A_FLOATS;
            const int L = ((lo % 4) + 4) % 4;
            const int RT = (((4 - L) % 4) + 1) % 4;
            const int wsB = TRANS ? (o0 - lo - (KD - 1) - RT) : (o0 + lo - L);      // first dense row of the window, a multiple of 4
            const int wsA = TRANS ? wsB : o0;
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;"
                         ::"r"(r_u32(full + s)), "r"(stage_bytes<TRANS>()) : "memory");
#pragma unroll
            for (int b = 0; b < 2; b++) {
                asm volatile(
                    "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                    ::"r"(r_u32(As + b * KD * abox<TRANS>())), "l"(&mapA), "r"(wsA + b * abox<TRANS>()), "r"(slot0),
                      "r"(r_u32(full + s)) : "memory");
                asm volatile(
                    "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                    ::"r"(r_u32(Bs + b * CG * BOXR)), "l"(&mapB), "r"(wsB + b * BOXR), "r"(c0), "r"(r_u32(full + s)) : "memory");
            }
            n++;
        }
        // the block's shared memory must outlive the copies in flight: wait (bounded) for the last stages issued
        for (int m = max(0, n - NS); m < n; m++) r_wait(full + (m % NS), (m / NS) & 1);
        return;
    }

    // ---- consumers: row thread rt owns rows 4*rt.., column half ch the columns 8*ch.. of the block's 16 ----
    const int rt = tid % ROWTHREADS, ch = tid / ROWTHREADS;
    const int i0 = o0 + 4 * rt;
    const int cb = c0 + ch * CT;                           // first column of this thread
    const int ncl = max(0, min(CT, P.ncols - cb));         // columns of this thread that exist
    float acc[CT][4];
#pragma unroll
    for (int c = 0; c < CT; c++)
#pragma unroll
        for (int j = 0; j < 4; j++) {
            acc[c][j] = 0.f;
            if (P.fc != 0.f && c < ncl && i0 + j < rows_out)
                acc[c][j] = __fmul_rn(P.C[(size_t)(cb + c) * P.ldc + i0 + j], P.fc);
        }
    int hoff[NW];
#pragma unroll
    for (int v = 0; v < NW; v++) {
        const int r = 4 * rt + 4 * v, b = r >= BOXR ? 1 : 0;
        hoff[v] = (b * CG + ch * CT) * BOXR + (r - b * BOXR);
    }
    if (reachable) {
        int n = 0;
        int4 d = ld_desc(P.passes);
        for (int p = 0; p < P.npass; p++) {
            const int lo = d.y, cnt = d.z;
            if (p + 1 < P.npass) d = ld_desc(P.passes + p + 1);        // the next descriptor is in flight during this pass
            if (!touches(lo, cnt)) continue;
            const int s = n % NS;
            if (!r_wait(full + s, (n / NS) & 1)) { if (P.status) *P.status = 6; return; }
            const float* As = sm + s * STAGE_FLOATS;
            const float* Bs = As + A_FLOATS;
            const int L = ((lo % 4) + 4) % 4;
            // block-uniform: all 8 diagonals present and every cell of the block's rows inside the matrix
            const bool interior = cnt == KD && o0 + TR <= rows_out &&
                                  (TRANS ? (o0 - lo - (KD - 1) >= 0 && o0 + TR - 1 - lo < P.h)
                                         : (o0 + lo >= 0 && o0 + TR - 1 + lo + (KD - 1) < P.w));
#define RUNS_GO(LV)                                                                                        \
            do {                                                                                           \
                if (interior) runs_pass<TRANS, EXACT, LV, true>(As, Bs, acc, hoff, rt, ncl, P, i0, lo, cnt);    \
                else runs_pass<TRANS, EXACT, LV, false>(As, Bs, acc, hoff, rt, ncl, P, i0, lo, cnt);           \
            } while (0)
            switch (L) { case 0: RUNS_GO(0); break; case 1: RUNS_GO(1); break; case 2: RUNS_GO(2); break; default: RUNS_GO(3); break; }
#undef RUNS_GO
            __syncwarp();
            if ((tid & 31) == 0)
                asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(r_u32(empty + s)) : "memory");
            n++;
        }
    }
    if (i0 >= rows_out) return;
    const bool vec_c = i0 + 4 <= rows_out && (P.ldc & 3) == 0 && (reinterpret_cast<uintptr_t>(P.C) & 15) == 0;
#pragma unroll
    for (int c = 0; c < CT; c++) {
        if (c >= ncl) continue;
        float* cp = P.C + (size_t)(cb + c) * P.ldc + i0;
        if (vec_c) {
            *reinterpret_cast<float4*>(cp) = make_float4(acc[c][0], acc[c][1], acc[c][2], acc[c][3]);
        } else {
#pragma unroll
            for (int j = 0; j < 4; j++)
                if (i0 + j < rows_out) cp[j] = acc[c][j];
        }
    }
}

static inline bool al16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// Row factor 1, diagonals mostly in runs (the plan found on average at least four per pass), 16-byte
// aligned operands.
bool prod_runs_applicable(const cuvdia_plan* p, const float* A, const float* B, int ldb) {
    return p->is_runs && p->d_passes != nullptr && al16(A) && al16(B) && p->stride % 4 == 0 && ldb % 4 == 0 &&
           tma_available();
}

template <bool TRANS, bool EXACT>
static int launch_runs_t(const cuvdia_plan* p, const float* A, const float* B, int ldb, float* C, int ldc, int ncols,
                         float fa, float fc, cudaStream_t st) {
    using namespace pr;
    CUtensorMap mapA, mapB;
    int rc = make_map_2d(&mapA, A, p->h, p->nd, p->stride, abox<TRANS>(), KD);
    if (rc) return rc;
    rc = make_map_2d(&mapB, B, TRANS ? p->h : p->w, ncols, ldb, BOXR, CG);
    if (rc) return rc;
    RunsParams P;
    P.h = p->h; P.w = p->w; P.ldc = ldc; P.ncols = ncols; P.npass = p->npass;
    P.off_min = p->off_min; P.off_max = p->off_max; P.fa = fa; P.fc = fc; P.C = C;
    P.passes = reinterpret_cast<const int4*>(p->d_passes);
    P.status = p->d_status;
    const int rows_out = TRANS ? p->w : p->h;
    const long long row_blocks = ((long long)rows_out + TR - 1) / TR;
    const long long blocks = row_blocks * ((ncols + CG - 1) / CG);
    if (blocks > 2147483647LL) { set_last_error("too many blocks"); return CUVDIA_ERR_UNSUPPORTED; }
    static bool attr[64] = {false};
    rc = allow_dynamic_smem(prod_runs_kernel<TRANS, EXACT>, SMEM, attr);
    if (rc) return rc;
    prod_runs_kernel<TRANS, EXACT><<<(unsigned)blocks, THREADS, SMEM, st>>>(mapA, mapB, P);
    count_launch();
    return check_launch("prod_runs_kernel");
}

int launch_prod_runs(const cuvdia_plan* p, const float* A, const float* B, int ldb, float* C, int ldc, int ncols,
                     bool trans, float fa, float fc, int mode, cudaStream_t st) {
    const bool exact = mode == CUVDIA_MODE_EXACT;
    if (trans) return exact ? launch_runs_t<true, true>(p, A, B, ldb, C, ldc, ncols, fa, fc, st)
                            : launch_runs_t<true, false>(p, A, B, ldb, C, ldc, ncols, fa, fc, st);
    return exact ? launch_runs_t<false, true>(p, A, B, ldb, C, ldc, ncols, fa, fc, st)
                 : launch_runs_t<false, false>(p, A, B, ldb, C, ldc, ncols, fa, fc, st);
}

}  // namespace cuvdia
