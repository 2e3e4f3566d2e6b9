// densedense_to_dia for scattered diagonal patterns (any row factor) whose neighbouring offsets lie
// close enough that a window of the second dense operand fits in shared memory.
//
//   C_dia[k][i] = factC*C_dia[k][i] + factAB * sum_b A[i,b] * B[i/rf + off_k, b]
//
// Every stored cell is a dot product over the batch between a row of A and a row of B; with
// scattered offsets no two cells of a thread share a B row, so B values cannot be reused from
// registers and the ceiling is one shared-memory word per multiply-add (a quarter of the FP32
// rate).  What can be saved is everything around that word:
//  * The diagonals are taken in ascending order of their offsets.  For a tile of 512 rows (256 where
//    two rows per thread do not apply) only the diagonals that have a cell inside the matrix on
//    some row of the tile are looked at - a contiguous range in that order - and they are cut into
//    groups of up to 16 whose B rows fit the staged window.  The (tile, group) pairs are listed once
//    per plan; a block owns one pair and one share of the batch.  With offsets spread over +-w/2 a
//    quarter of all (row, diagonal) pairs lie outside the matrix, most of them in whole groups that
//    are never scheduled.
//  * Per chunk of batch columns a block needs its tile of A and the window of B rows the group can
//    touch (rows i/rf + off_min .. off_max of the group; rows outside B arrive as zeros).  One
//    producer warp brings both in with TMA tile loads (cp.async.bulk.tensor, no multicast) of
//    256 rows x 1 column each, into a ring of stages guarded by full/empty mbarriers with bounded
//    waits; the eight consumer warps never meet a block barrier and issue nothing but shared-memory
//    loads and multiply-adds: a staged B value serves about five cells, each thread keeps 32
//    running sums (two rows x 16 diagonals).
//  * The batch split is chosen so that the blocks fill whole waves of two blocks per SM.
// The batch is summed in column order within a split and the splits in order by a second kernel,
// so the result does not depend on scheduling.  Only cells inside a diagonal's valid range are
// written (matrix_ops/densedense_to_sparse.cu:104-119).
#include <cuda.h>

#include "cuvdia_internal.cuh"

namespace cuvdia {

int make_map_2d(CUtensorMap* m, const float* base, long long dim0, long long dim1, long long pitch, int box0, int box1);
int launch_dd2dia_combine(const cuvdia_plan* p, float* Cv, float fa, float fc, int nsplit, const float* partial,
                          cudaStream_t st);

namespace dw {
constexpr int CONSUMERS = 256;       // threads that do the arithmetic; one more warp issues the copies
constexpr int THREADS = CONSUMERS + 32;
constexpr int KG = 16;               // diagonals per group
constexpr int BOX = 256;             // rows per TMA box
constexpr int NBOX = 5;              // boxes per staged B column: the window holds 1280 rows
constexpr int WCAP = NBOX * BOX;
constexpr int BC = 4;                // batch columns per stage (4 x 3 stages measured best of the shapes that leave two blocks per SM)
constexpr int STAGES = 3;
constexpr unsigned SPIN_LIMIT = 1u << 26;
template <int RPT> __host__ __device__ constexpr int stage_floats() { return BC * (RPT * CONSUMERS + WCAP); }
template <int RPT> constexpr size_t smem_bytes() { return sizeof(float) * STAGES * stage_floats<RPT>() + 64; }
}  // namespace dw

struct DdWindowParams {
    int h, w, nd, S, rf;
    int ncols, nsplit;
    float fa, fc;
    float* C; float* partial;
    const int* sorted_slot;          // storage slot of the k-th smallest offset
    const int* sorted_off;           // the k-th smallest offset
    const int* items;                // (first row of the tile, first diagonal in offset order, diagonals) per block
    int* status;
};

__device__ __forceinline__ unsigned dw_smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ bool dw_wait(unsigned long long* bar, unsigned parity, unsigned limit) {
    const unsigned addr = dw_smem_u32(bar);
    for (unsigned it = 0; it < limit; it++) {
        unsigned done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done) : "r"(addr), "r"(parity) : "memory");
        if (done) return true;
    }
    return false;
}

// RPT: rows per thread (2 where the row factor divides 256, so that the second row's cells sit a constant distance
// from the first's).  The stage size and the pitch of a staged column are compile-time constants and the ring is
// walked with a compile-time stage index, so that a cell's shared-memory address is a register plus an immediate.
template <int RPT>
__global__ void __launch_bounds__(dw::THREADS, 2)
dd2dia_window_kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB,
                     const DdWindowParams P) {
    using namespace dw;
    constexpr int TR = RPT * CONSUMERS;              // rows per block
    constexpr int STAGE = stage_floats<RPT>();       // A tile [BC][TR], then B window [BC][WCAP]
    extern __shared__ __align__(1024) float smem[];
    unsigned long long* const full = reinterpret_cast<unsigned long long*>(smem + STAGES * STAGE);
    unsigned long long* const empty = full + STAGES;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int i0 = P.items[3 * blockIdx.x], g0 = P.items[3 * blockIdx.x + 1], gn = P.items[3 * blockIdx.x + 2];
    const int z = blockIdx.y;
    const int nch_all = (P.ncols + BC - 1) / BC;
    const int ch0 = (int)((long long)nch_all * z / P.nsplit), ch1 = (int)((long long)nch_all * (z + 1) / P.nsplit);
    const int nch = ch1 - ch0;
    const int gmin = P.sorted_off[g0], gmax = P.sorted_off[g0 + gn - 1];
    const int wbase = (i0 / P.rf + gmin) & ~3;       // first staged B row: the window's first row rounded down to 4
    const int nbox = ((i0 + TR - 1) / P.rf + gmax - wbase) / BOX + 1;      // boxes that hold rows a cell can touch

    if (tid == 0) {
#pragma unroll
        for (int s = 0; s < STAGES; s++) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(dw_smem_u32(&full[s])));
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(dw_smem_u32(&empty[s])), "r"(CONSUMERS / 32));
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    if (warp == CONSUMERS / 32) {
        // ---- producer warp: per chunk BC * (RPT + nbox) boxes of 256 rows x 1 column, spread over the lanes ----
        const int nops = BC * (RPT + nbox);
        const unsigned tx = sizeof(float) * BOX * (unsigned)nops;
        for (int c = 0; c < nch; c++) {
            const int s = c % STAGES;
            bool ok = true;
            if (c >= STAGES && lane == 0) ok = dw_wait(&empty[s], ((c / STAGES) - 1) & 1, SPIN_LIMIT);
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) {
                // the consumers never handed the stage back: record it, wait (bounded) for the copies already under
                // way so that none lands in shared memory the block has given back, and stop
                if (lane == 0) {
                    *P.status = 7;
                    for (int c2 = max(0, c - STAGES); c2 < c; c2++) dw_wait(&full[c2 % STAGES], (c2 / STAGES) & 1, 1u << 22);
                }
                return;
            }
            const unsigned bar = dw_smem_u32(&full[s]);
            if (lane == 0)
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(tx) : "memory");
            __syncwarp();
            const int col0 = (ch0 + c) * BC;
            float* const st = smem + s * STAGE;
            for (int op = lane; op < nops; op += 32) {
                const int col = op % BC, q = op / BC;
                if (q < RPT)
                    asm volatile(
                        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                        ::"r"(dw_smem_u32(st + col * TR + q * BOX)), "l"(&mapA), "r"(i0 + q * BOX), "r"(col0 + col), "r"(bar)
                        : "memory");
                else
                    asm volatile(
                        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                        ::"r"(dw_smem_u32(st + BC * TR + col * WCAP + (q - RPT) * BOX)), "l"(&mapB),
                          "r"(wbase + (q - RPT) * BOX), "r"(col0 + col), "r"(bar)
                        : "memory");
            }
        }
        return;
    }

    // ---- consumers ----
    // word index of the cells of this thread's first row inside stage 0 (indices into the shared array itself, so
    // that the loads below stay in the shared address space); the second row's cells lie roff words further
    const int roff = CONSUMERS / P.rf;
    int cell[KG];
#pragma unroll
    for (int kk = 0; kk < KG; kk++) {
        const int off = kk < gn ? P.sorted_off[g0 + kk] : gmin;
        cell[kk] = BC * TR + ((i0 + tid) / P.rf + off - wbase);
    }
    float acc[RPT][KG];
#pragma unroll
    for (int r = 0; r < RPT; r++)
#pragma unroll
        for (int kk = 0; kk < KG; kk++) acc[r][kk] = 0.f;

    for (int cb = 0; cb < nch; cb += STAGES) {
#pragma unroll
        for (int s = 0; s < STAGES; s++) {
            if (cb + s >= nch) break;
            if (!dw_wait(&full[s], (cb / STAGES) & 1, SPIN_LIMIT)) { *P.status = 7; return; }
            const float* st = smem + s * STAGE;
            const float* st2 = st + roff;
#pragma unroll
            for (int c = 0; c < BC; c++) {
                const float a0 = st[c * TR + tid];
                const float a1 = RPT == 2 ? st[c * TR + CONSUMERS + tid] : 0.f;
#pragma unroll
                for (int kk = 0; kk < KG; kk++) {
                    acc[0][kk] = fmaf(a0, st[cell[kk] + c * WCAP], acc[0][kk]);
                    if (RPT == 2) acc[RPT - 1][kk] = fmaf(a1, st2[cell[kk] + c * WCAP], acc[RPT - 1][kk]);
                }
            }
            // hand the stage back: one arrival per warp
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(dw_smem_u32(&empty[s])) : "memory");
        }
    }

#pragma unroll
    for (int r = 0; r < RPT; r++) {
        const int i = i0 + r * CONSUMERS + tid;
        if (i >= P.h) continue;
#pragma unroll
        for (int kk = 0; kk < KG; kk++) {
            if (kk >= gn) break;
            const int jj = i / P.rf + P.sorted_off[g0 + kk];
            if (jj < 0 || jj >= P.w) continue;
            const size_t cellidx = (size_t)P.sorted_slot[g0 + kk] * P.S + i;
            if (P.nsplit == 1) {
                float s = acc[r][kk];
                if (P.fa != 1.f) s = __fmul_rn(P.fa, s);
                P.C[cellidx] = (P.fc != 0.f) ? __fadd_rn(__fmul_rn(P.fc, P.C[cellidx]), s) : s;
            } else {
                P.partial[(size_t)z * P.nd * P.S + cellidx] = acc[r][kk];
            }
        }
    }
}

// Rows per thread for this plan: two where the row factor divides 256 and the matrix has rows to fill the GPU
// with such tiles.
static int window_rpt(int h, int rf) { return (dw::CONSUMERS % rf == 0 && h >= 4 * 2 * dw::CONSUMERS) ? 2 : 1; }

// The (tile, group) pairs of a plan: for every tile of rows the diagonals that have a cell inside the matrix on
// some row of the tile - a contiguous range in ascending offset order - cut greedily into groups of up to 16 whose
// B rows fit the staged window.  sorted_off: the offsets in ascending order.  Three ints per pair.
void window_items(int h, int w, int nd, int rf, const int* sorted_off, std::vector<int>* items) {
    using namespace dw;
    const int TR = window_rpt(h, rf) * CONSUMERS;
    items->clear();
    for (int i0 = 0; i0 < h; i0 += TR) {
        const int q0 = i0 / rf, q1 = (std::min(h, i0 + TR) - 1) / rf;          // dense rows of the tile before the offset
        const int qt = (i0 + TR - 1) / rf;                                     // the same for a full tile (what is staged)
        // diagonal k has a cell inside the matrix iff q1 + off >= 0 and q0 + off < w
        int klo = (int)(std::lower_bound(sorted_off, sorted_off + nd, -q1) - sorted_off);
        int khi = (int)(std::lower_bound(sorted_off, sorted_off + nd, w - q0) - sorted_off);
        for (int k = klo; k < khi;) {
            const int wbase = (q0 + sorted_off[k]) & ~3;
            int n = 1;
            while (n < KG && k + n < khi && qt + sorted_off[k + n] - wbase < WCAP) n++;
            items->push_back(i0); items->push_back(k); items->push_back(n);
            k += n;
        }
    }
}

// 16-byte aligned operands, TMA, enough work to stage for, and groups that are not mostly padding: at least half of
// the 16 places of a group filled on average.
bool dd2dia_window_applicable(const cuvdia_plan* p, const float* A, int lda, const float* B, int ldb, int ncols) {
    auto al16 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
    if (!(al16(A) && al16(B) && lda % 4 == 0 && ldb % 4 == 0)) return false;
    return p->d_witems != nullptr && p->n_witems > 0 && p->witem_diagonals >= 8LL * p->n_witems && p->nd >= 16 &&
           ncols >= 32 && tma_available();
}

// Batch shares: enough blocks for whole waves of two per SM; among the shares that fill their last wave about as
// well as the best one the smallest, since every share costs a pass of the second kernel over its partial sums
// (config 2, 56 pairs: 5 shares 80 us; 4: 96, 6: 112, 8: 95, 10: 83).
static int window_nsplit(long long items, int ncols) {
    const long long slots = 2LL * sm_count();
    const int smax = std::max(1, std::min(64, ncols / 64));
    if (items >= 4 * slots) return 1;
    double best = 0.0;
    std::vector<double> eff(smax + 1, 0.0);
    for (int s = 1; s <= smax; s++) {
        const long long ctas = items * s, waves = (ctas + slots - 1) / slots;
        eff[s] = (double)ctas / (double)(waves * slots);
        best = std::max(best, eff[s]);
    }
    for (int s = 1; s <= smax; s++)
        if (eff[s] >= best - 0.04) return s;
    return 1;
}

int launch_dd2dia_window(cuvdia_plan* p, float* Cv, const float* A, int lda, const float* B, int ldb, int ncols,
                         float fa, float fc, cudaStream_t st) {
    using namespace dw;
    if (!p->d_witems || p->n_witems <= 0) { set_last_error("window does not fit"); return CUVDIA_ERR_UNSUPPORTED; }
    CUtensorMap mapA, mapB;
    int rc = make_map_2d(&mapA, A, p->h, ncols, lda, BOX, 1);
    if (rc) return rc;
    rc = make_map_2d(&mapB, B, p->w, ncols, ldb, BOX, 1);
    if (rc) return rc;
    DdWindowParams P;
    P.h = p->h; P.w = p->w; P.nd = p->nd; P.S = p->stride; P.rf = p->rf;
    P.ncols = ncols;
    P.fa = fa; P.fc = fc; P.C = Cv;
    P.sorted_slot = p->d_sorted; P.sorted_off = p->d_sorted + p->nd;
    P.items = p->d_witems; P.status = p->d_status;
    const int RPT = window_rpt(p->h, p->rf);
    const int nsplit = window_nsplit(p->n_witems, ncols);
    P.nsplit = nsplit;
    P.partial = nullptr;
    if (nsplit > 1) {
        rc = ensure_plan_scratch(p, (size_t)nsplit * p->nd * p->stride, st);
        if (rc) return rc;
        P.partial = p->scratch;
    }
#define DW_GO(RV)                                                                                      \
    do {                                                                                               \
        static bool attr[64] = {false};                                                                \
        rc = allow_dynamic_smem(dd2dia_window_kernel<RV>, smem_bytes<RV>(), attr);                     \
        if (rc) return rc;                                                                             \
        dd2dia_window_kernel<RV><<<dim3(p->n_witems, nsplit), THREADS, smem_bytes<RV>(), st>>>(mapA, mapB, P); \
    } while (0)
    if (RPT == 2) DW_GO(2); else DW_GO(1);
#undef DW_GO
    count_launch();
    rc = check_launch("dd2dia_window_kernel");
    if (rc) return rc;
    if (nsplit > 1) rc = launch_dd2dia_combine(p, Cv, fa, fc, nsplit, P.partial, st);
    return rc;
}

}  // namespace cuvdia
