// densedense_to_dia for long, narrow bands (row_fact 1, at most 16 consecutive diagonals): the
// memory-bound regime, where A and B should cross HBM once and the dense-tile kernel of
// dd2dia_band.cu would spend 128/num_dia of its arithmetic outside the band.
//
//   G[k][i] = factC*G[k][i] + factAB * sum_b A[i,b] * B[i+lo+k, b]
//
// A block owns 512 rows (4 per thread) and all diagonals; it walks the batch 16 columns at a time.
// Per round one thread issues eight TMA tile loads (cp.async.bulk.tensor, no multicast) - the
// 512 x 16 tile of A and the 544 x 16 window of B - onto one mbarrier (bounded wait); three blocks
// share an SM, so loads and arithmetic of different blocks overlap.  Per batch column a thread
// reads its 4 values of A and the 19 B rows its 4 x 16 cells touch with aligned 128-bit shared
// loads into a register window (cell (row j, diagonal k) uses entry L + j + k; L, the alignment of
// the first offset, is a template parameter, so the indices are compile-time) and issues 64 fused
// multiply-adds into 64 accumulators.  The batch is summed in column order by one thread per cell,
// so results are bit-reproducible.  Cells outside a diagonal's range are never touched.
//
// The same block also serves patterns made of RUNS of consecutive diagonals - convolution-pattern matrices
// (basics/filter_factory.hpp:43-76; the reference's speed fixture src/tests/densedense_to_dia_speed.cpp:65-106): the plan
// cuts the offset list, in storage order, into passes of up to 8 consecutive diagonals, and dd2dia_runs_kernel runs
// one block per row tile and pass, a narrow band of its own (8 diagonals x 4 rows = 32 running sums per thread, a
// 16-entry register window).  The alignment of a pass's first offset differs from pass to pass, so the block picks
// its instantiation at run time (block-uniform).
#include <cuda.h>

#include "cuvdia_internal.cuh"

namespace cuvdia {

int make_map_2d(CUtensorMap* m, const float* base, long long dim0, long long dim1, long long pitch, int box0, int box1);

namespace ds {
constexpr int THREADS = 128;
constexpr int TR = 4 * THREADS;       // rows per block
constexpr int KD = 16;                // diagonals (all of them)
constexpr int NC = 16;                // batch columns per round
constexpr int XBOX = 128, HBOX = 136; // rows per TMA box (4 boxes each)
constexpr int X_FLOATS = 4 * NC * XBOX;
constexpr int H_FLOATS = 4 * NC * HBOX;
constexpr size_t SMEM = sizeof(float) * (X_FLOATS + H_FLOATS) + 64;
constexpr unsigned SPIN_LIMIT = 1u << 26;
}

struct DdStreamParams {
    int h, w, nd, lo, S, ncols;
    float fa, fc;
    float* G;
    int* status;
};

__device__ __forceinline__ unsigned ds_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }

// One block: rows o0 .. o0+511, diagonals slot0 .. slot0+cnt-1 (cnt <= KD) whose offsets are lo, lo+1, ...
// NV = 128-bit loads per B column: 4*NV window entries >= L + 3 + KD.
template <int L, int KD, int NV>
__device__ __forceinline__ void dd_stream_block(const CUtensorMap& mapA, const CUtensorMap& mapB, const DdStreamParams& P,
                                                const int slot0, const int lo, const int cnt) {
    using namespace ds;
    extern __shared__ __align__(1024) float sm[];
    float* const Xs = sm;                       // [4][NC][XBOX]
    float* const Hs = sm + X_FLOATS;            // [4][NC][HBOX]
    unsigned long long* const bar = reinterpret_cast<unsigned long long*>(sm + X_FLOATS + H_FLOATS);
    const int tid = threadIdx.x;
    const int o0 = blockIdx.x * TR;
    const int i0 = o0 + 4 * tid;
    const int wsH = o0 + lo - L;                // first matrix row of the B window, a multiple of 4
    if (tid == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(ds_u32(bar)));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    float acc[KD][4];
#pragma unroll
    for (int k = 0; k < KD; k++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[k][j] = 0.f;

    // this thread's words inside the boxes: A rows 4*tid.., B window rows 4*tid + 4v
    const int xb = (4 * tid) / XBOX, xr = (4 * tid) % XBOX;
    int hoff[NV];
#pragma unroll
    for (int v = 0; v < NV; v++) {
        const int r = 4 * tid + 4 * v;
        const int b = r / HBOX;
        hoff[v] = b * NC * HBOX + (r - b * HBOX);
    }

    unsigned phase = 0;
    for (int cbase = 0; cbase < P.ncols; cbase += NC) {
        if (tid == 0) {
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;"
                         ::"r"(ds_u32(bar)), "r"((unsigned)(sizeof(float) * (X_FLOATS + H_FLOATS))) : "memory");
#pragma unroll
            for (int b = 0; b < 4; b++) {
                asm volatile(
                    "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                    ::"r"(ds_u32(Xs + b * NC * XBOX)), "l"(&mapA), "r"(o0 + b * XBOX), "r"(cbase), "r"(ds_u32(bar)) : "memory");
                asm volatile(
                    "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                    ::"r"(ds_u32(Hs + b * NC * HBOX)), "l"(&mapB), "r"(wsH + b * HBOX), "r"(cbase), "r"(ds_u32(bar)) : "memory");
            }
        }
        bool done = false;
        for (unsigned it = 0; it < SPIN_LIMIT && !done; it++) {
            unsigned d;
            asm volatile(
                "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                : "=r"(d) : "r"(ds_u32(bar)), "r"(phase) : "memory");
            done = d != 0;
        }
        if (!done) { if (P.status) *P.status = 4; return; }
        phase ^= 1;
        // columns past the batch arrive as zeros and add nothing
#pragma unroll 2
        for (int c = 0; c < NC; c++) {
            const float4 x4 = *reinterpret_cast<const float4*>(Xs + (xb * NC + c) * XBOX + xr);
            const float x[4] = {x4.x, x4.y, x4.z, x4.w};
            float wv[4 * NV];
#pragma unroll
            for (int v = 0; v < NV; v++) {
                const float4 t = *reinterpret_cast<const float4*>(Hs + hoff[v] + c * HBOX);
                wv[4 * v] = t.x; wv[4 * v + 1] = t.y; wv[4 * v + 2] = t.z; wv[4 * v + 3] = t.w;
            }
#pragma unroll
            for (int k = 0; k < KD; k++)
#pragma unroll
                for (int j = 0; j < 4; j++) acc[k][j] = fmaf(x[j], wv[L + j + k], acc[k][j]);
        }
        __syncthreads();          // the tiles may be overwritten by the next round's loads
    }

    // ---- store: G[k][i0..i0+3], only cells inside the matrix ----
    const bool vec = i0 + 4 <= P.h && i0 + lo >= 0 && i0 + 3 + lo + (cnt - 1) < P.w;   // all 4 x cnt cells valid
#pragma unroll
    for (int k = 0; k < KD; k++) {
        if (k >= cnt) break;
        float* gp = P.G + (size_t)(slot0 + k) * P.S + i0;
        float v[4];
#pragma unroll
        for (int j = 0; j < 4; j++) v[j] = (P.fa != 1.f) ? __fmul_rn(P.fa, acc[k][j]) : acc[k][j];
        if (vec) {
            float4 o = make_float4(v[0], v[1], v[2], v[3]);
            if (P.fc != 0.f) {
                const float4 g = *reinterpret_cast<const float4*>(gp);
                o.x = __fadd_rn(__fmul_rn(P.fc, g.x), v[0]); o.y = __fadd_rn(__fmul_rn(P.fc, g.y), v[1]);
                o.z = __fadd_rn(__fmul_rn(P.fc, g.z), v[2]); o.w = __fadd_rn(__fmul_rn(P.fc, g.w), v[3]);
            }
            *reinterpret_cast<float4*>(gp) = o;
        } else {
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const int jb = i0 + j + lo + k;
                if (i0 + j < P.h && jb >= 0 && jb < P.w)
                    gp[j] = (P.fc != 0.f) ? __fadd_rn(__fmul_rn(P.fc, gp[j]), v[j]) : v[j];
            }
        }
    }
}

template <int L>
__global__ void __launch_bounds__(ds::THREADS, 3)
dd2dia_stream_kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB,
                     const DdStreamParams P) {
    dd_stream_block<L, ds::KD, 6>(mapA, mapB, P, 0, P.lo, P.nd);
}

// Runs of consecutive diagonals: blockIdx.y = pass (first slot, first offset, count <= 8) of the plan's pass list.
__global__ void __launch_bounds__(ds::THREADS, 3)
dd2dia_runs_kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB,
                   const DdStreamParams P, const int* __restrict__ passes) {
    const int slot0 = passes[4 * blockIdx.y], lo = passes[4 * blockIdx.y + 1], cnt = passes[4 * blockIdx.y + 2];
    switch (((lo % 4) + 4) % 4) {                      // block-uniform
        case 0: dd_stream_block<0, 8, 4>(mapA, mapB, P, slot0, lo, cnt); break;
        case 1: dd_stream_block<1, 8, 4>(mapA, mapB, P, slot0, lo, cnt); break;
        case 2: dd_stream_block<2, 8, 4>(mapA, mapB, P, slot0, lo, cnt); break;
        default: dd_stream_block<3, 8, 4>(mapA, mapB, P, slot0, lo, cnt); break;
    }
}

static inline bool al16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

bool dd2dia_runs_applicable(const cuvdia_plan* p, const float* Cv, const float* A, int lda, const float* B, int ldb,
                            int ncols) {
    // passes of 8 consecutive diagonals on average at least half full, enough blocks to be worth the TMA set-up
    return p->is_runs && p->d_passes != nullptr && p->rf == 1 && ncols >= 1 && al16(A) && al16(B) && al16(Cv) &&
           lda % 4 == 0 && ldb % 4 == 0 && p->stride % 4 == 0 && tma_available() &&
           (long long)((p->h + ds::TR - 1) / ds::TR) * p->npass >= 16;
}

int launch_dd2dia_runs(cuvdia_plan* p, float* Cv, const float* A, int lda, const float* B, int ldb, int ncols,
                       float fa, float fc, cudaStream_t st) {
    using namespace ds;
    CUtensorMap mapA, mapB;
    int rc = make_map_2d(&mapA, A, p->h, ncols, lda, XBOX, NC);
    if (rc) return rc;
    rc = make_map_2d(&mapB, B, p->w, ncols, ldb, HBOX, NC);
    if (rc) return rc;
    DdStreamParams P;
    P.h = p->h; P.w = p->w; P.nd = p->nd; P.lo = 0; P.S = p->stride; P.ncols = ncols;
    P.fa = fa; P.fc = fc; P.G = Cv; P.status = p->d_status;
    const int blocks = (p->h + TR - 1) / TR;
    if (p->npass > 65535) { set_last_error("too many runs of diagonals"); return CUVDIA_ERR_UNSUPPORTED; }
    static bool attr[64] = {false};
    rc = allow_dynamic_smem(dd2dia_runs_kernel, SMEM, attr);
    if (rc) return rc;
    dd2dia_runs_kernel<<<dim3(blocks, p->npass), THREADS, SMEM, st>>>(mapA, mapB, P, p->d_passes);
    count_launch();
    return check_launch("dd2dia_runs_kernel");
}

bool dd2dia_stream_applicable(const cuvdia_plan* p, const float* Cv, const float* A, int lda, const float* B, int ldb,
                              int ncols) {
    return p->is_band && p->rf == 1 && p->nd <= ds::KD && p->h >= 64 * ds::TR && ncols >= 1 && al16(A) && al16(B) &&
           al16(Cv) && lda % 4 == 0 && ldb % 4 == 0 && p->stride % 4 == 0 && tma_available();
}

int launch_dd2dia_stream(cuvdia_plan* p, float* Cv, const float* A, int lda, const float* B, int ldb, int ncols,
                         float fa, float fc, cudaStream_t st) {
    using namespace ds;
    CUtensorMap mapA, mapB;
    int rc = make_map_2d(&mapA, A, p->h, ncols, lda, XBOX, NC);
    if (rc) return rc;
    rc = make_map_2d(&mapB, B, p->w, ncols, ldb, HBOX, NC);
    if (rc) return rc;
    DdStreamParams P;
    P.h = p->h; P.w = p->w; P.nd = p->nd; P.lo = p->band_lo; P.S = p->stride; P.ncols = ncols;
    P.fa = fa; P.fc = fc; P.G = Cv; P.status = p->d_status;
    const int blocks = (p->h + TR - 1) / TR;
    const int L = ((p->band_lo % 4) + 4) % 4;
#define GO(LV)                                                                              \
    do {                                                                                    \
        static bool attr[64] = {false};                                                     \
        rc = allow_dynamic_smem(dd2dia_stream_kernel<LV>, SMEM, attr);                      \
        if (rc) return rc;                                                                  \
        dd2dia_stream_kernel<LV><<<blocks, THREADS, SMEM, st>>>(mapA, mapB, P);             \
    } while (0)
    switch (L) { case 0: GO(0); break; case 1: GO(1); break; case 2: GO(2); break; default: GO(3); break; }
#undef GO
    count_launch();
    return check_launch("dd2dia_stream_kernel");
}

}  // namespace cuvdia
