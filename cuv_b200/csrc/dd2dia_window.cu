// densedense_to_dia for scattered diagonal patterns (any row factor) whose neighbouring offsets lie
// close enough that a window of the second dense operand fits in shared memory.
//
//   C_dia[k][i] = factC*C_dia[k][i] + factAB * sum_b A[i,b] * B[i/rf + off_k, b]
//
// Every stored cell is a dot product over the batch between a row of A and a row of B; with
// scattered offsets no two cells of a thread share a B row, so B values cannot be reused from
// registers and the ceiling is one shared-memory word per multiply-add (a quarter of the FP32
// rate).  What can be saved is the traffic behind it: the plain kernel fetches every B value from
// L2 once per cell.  Here the diagonals are taken in ascending order of their offsets, 32 (or 16) at a
// time; a block owns 256 rows and one such group, and stages, per 8 batch columns, its 256 x 8
// tile of A and the window of B rows the group can touch (rows i/rf + off_min .. off_max of the
// group; rows outside B arrive as zeros) with 16-byte asynchronous copies, one chunk ahead of the
// arithmetic (two stages).  A staged B value then serves
// every cell of the block on its row - about 256*32/window times - and each thread keeps 32
// running sums.  Several blocks share an SM, so one block's copies overlap another's arithmetic.
// The batch is summed in column order within a split and the splits in order by a second kernel,
// so the result does not depend on scheduling.  Only cells inside a diagonal's valid range are
// written (matrix_ops/densedense_to_sparse.cu:104-119).
#include "cuvdia_internal.cuh"

namespace cuvdia {

namespace dw {
constexpr int THREADS = 256;         // rows per block
constexpr int BC = 8;                // batch columns per staged chunk
constexpr int PITCH = 1032;          // words per staged B column: two 41 KB stages, two blocks per SM
}

struct DdWindowParams {
    int h, w, nd, S, rf;
    int lda, ldb, ncols, nsplit;
    float fa, fc;
    const float* A; const float* B; float* C; float* partial;
    const int* sorted_slot;          // storage slot of the k-th smallest offset
    const int* sorted_off;           // the k-th smallest offset
};

// KG: diagonals per group (32, or 16 where 32 neighbours span too many rows for the window).  The pitch of a staged
// column is a compile-time constant, so that a cell's shared-memory address is a register plus an immediate.
template <int KG>
__global__ void __launch_bounds__(dw::THREADS, 2)
dd2dia_window_kernel(const DdWindowParams P) {
    using namespace dw;
    constexpr int STAGE = BC * (THREADS + PITCH);    // words per stage: A tile [BC][THREADS], B window [BC][PITCH]
    extern __shared__ __align__(16) float smem[];    // two stages
    const int tid = threadIdx.x;
    const int i0 = blockIdx.x * THREADS;
    const int g0 = blockIdx.y * KG;                  // first diagonal (in offset order) of the group
    const int gn = min(KG, P.nd - g0);
    const int z = blockIdx.z;
    const int b0 = (int)((long long)P.ncols * z / P.nsplit), b1 = (int)((long long)P.ncols * (z + 1) / P.nsplit);
    const int gmin = P.sorted_off[g0], gmax = P.sorted_off[g0 + gn - 1];
    const int i = i0 + tid;
    const int last = min(i0 + THREADS, P.h) - 1;     // last row of the block
    const int wbase = (i0 / P.rf + gmin) & ~3;       // first staged B row: the window's first row rounded down to 4
    const int wchunks = (last / P.rf + gmax - wbase + 4) / 4;      // 16-byte pieces per staged column

    // word index of this thread's 32 cells inside stage 0 (indices into the shared array itself, so that the
    // loads below stay in the shared address space)
    int cell[KG];
#pragma unroll
    for (int kk = 0; kk < KG; kk++) {
        const int off = kk < gn ? P.sorted_off[g0 + kk] : gmin;
        cell[kk] = BC * THREADS + (min(i, last) / P.rf + off - wbase);
    }
    float acc[KG];
#pragma unroll
    for (int kk = 0; kk < KG; kk++) acc[kk] = 0.f;

    const unsigned sm_u = (unsigned)__cvta_generic_to_shared(smem);
    // 16-byte asynchronous copies; bytes past the end of an operand (or of this split's columns) arrive as zeros.
    // What does not depend on the chunk is worked out once: this thread's piece of the A tile (two columns per
    // chunk half) and its pieces of a B column.
    const int qa = tid & (THREADS / 4 - 1), ca = tid / (THREADS / 4);      // A: piece qa of columns ca, ca+4
    const int rowa = i0 + 4 * qa;
    const unsigned bytes_a = 4u * (unsigned)max(0, min(4, P.h - rowa));
    const float* const srca = P.A + min(rowa, (P.h - 1) & ~3);
    const unsigned dsta = 4u * (unsigned)(ca * THREADS + 4 * qa);
    auto stage = [&](int buf, int cb) {
        const unsigned base = sm_u + 4u * (unsigned)(buf * STAGE);
#pragma unroll
        for (int u = 0; u < BC / 4; u++) {                                  // A tile
            const int c = ca + 4 * u;
            const bool col_ok = cb + c < b1;
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;"
                         ::"r"(base + dsta + 4u * (unsigned)(4 * u * THREADS)),
                           "l"(srca + (size_t)(col_ok ? cb + c : b0) * P.lda), "r"(col_ok ? bytes_a : 0u) : "memory");
        }
        for (int q = tid; q < wchunks; q += THREADS) {                      // B window: piece q of every column
            const int row = wbase + 4 * q;
            const unsigned bytes_b = row >= 0 ? 4u * (unsigned)max(0, min(4, P.w - row)) : 0u;
            const float* const srcb = P.B + min(max(row, 0), (P.w - 1) & ~3);
            const unsigned dstb = base + 4u * (unsigned)(BC * THREADS + 4 * q);
#pragma unroll
            for (int c = 0; c < BC; c++) {
                const bool col_ok = cb + c < b1;
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;"
                             ::"r"(dstb + 4u * (unsigned)(c * PITCH)), "l"(srcb + (size_t)(col_ok ? cb + c : b0) * P.ldb),
                               "r"(col_ok ? bytes_b : 0u) : "memory");
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };

    if (b0 < b1) stage(0, b0);
    int buf = 0;
    for (int cb = b0; cb < b1; cb += BC, buf ^= 1) {
        // the next chunk is fetched while this one is consumed
        if (cb + BC < b1) { stage(buf ^ 1, cb + BC); asm volatile("cp.async.wait_group 1;" ::: "memory"); }
        else asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();
        const float* st = smem + buf * STAGE;
        // ---- 8 columns x 32 cells per thread ----
#pragma unroll
        for (int c = 0; c < BC; c++) {
            const float a = st[c * THREADS + tid];
#pragma unroll
            for (int kk = 0; kk < KG; kk++) acc[kk] = fmaf(a, st[cell[kk] + c * PITCH], acc[kk]);
        }
        __syncthreads();                             // everyone is done with this stage before it is refilled
    }

    if (i >= P.h) return;
#pragma unroll
    for (int kk = 0; kk < KG; kk++) {
        if (kk >= gn) break;
        const int jj = i / P.rf + P.sorted_off[g0 + kk];
        if (jj < 0 || jj >= P.w) continue;
        const size_t cellidx = (size_t)P.sorted_slot[g0 + kk] * P.S + i;
        if (P.nsplit == 1) {
            float s = acc[kk];
            if (P.fa != 1.f) s = __fmul_rn(P.fa, s);
            P.C[cellidx] = (P.fc != 0.f) ? __fadd_rn(__fmul_rn(P.fc, P.C[cellidx]), s) : s;
        } else {
            P.partial[(size_t)z * P.nd * P.S + cellidx] = acc[kk];
        }
    }
}

int launch_dd2dia_combine(const cuvdia_plan* p, float* Cv, float fa, float fc, int nsplit, const float* partial,
                          cudaStream_t st);

// Diagonals per group for this plan: 32 if the rows such a group can touch fit the staged window, else 16, else 0.
static int window_group(const cuvdia_plan* p) {
    const int tile = (dw::THREADS - 1) / p->rf + 1;
    if (p->group_window_max[1] > 0 && tile + p->group_window_max[1] + 7 <= dw::PITCH) return 32;
    if (p->group_window_max[0] > 0 && tile + p->group_window_max[0] + 7 <= dw::PITCH) return 16;
    return 0;
}

// Neighbouring diagonals (in offset order) close enough for the window, 16-byte aligned operands, and enough work
// to stage for.
bool dd2dia_window_applicable(const cuvdia_plan* p, const float* A, int lda, const float* B, int ldb, int ncols) {
    auto al16 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
    if (!(al16(A) && al16(B) && lda % 4 == 0 && ldb % 4 == 0)) return false;
    return p->d_sorted != nullptr && window_group(p) != 0 && p->nd >= 16 && ncols >= 32;
}

int launch_dd2dia_window(cuvdia_plan* p, float* Cv, const float* A, int lda, const float* B, int ldb, int ncols,
                         float fa, float fc, cudaStream_t st) {
    using namespace dw;
    DdWindowParams P;
    P.h = p->h; P.w = p->w; P.nd = p->nd; P.S = p->stride; P.rf = p->rf;
    P.lda = lda; P.ldb = ldb; P.ncols = ncols;
    const int KG = window_group(p);
    if (KG == 0) { set_last_error("window does not fit"); return CUVDIA_ERR_UNSUPPORTED; }
    P.fa = fa; P.fc = fc; P.A = A; P.B = B; P.C = Cv;
    P.sorted_slot = p->d_sorted; P.sorted_off = p->d_sorted + p->nd;
    const int gx = (p->h + THREADS - 1) / THREADS, gy = (p->nd + KG - 1) / KG;
    if (gy > 65535) { set_last_error("num_dia too large for densedense_to_dia"); return CUVDIA_ERR_UNSUPPORTED; }
    int nsplit = 1;
    const long long ctas = (long long)gx * gy, want = 4LL * sm_count();
    if (ctas < want) nsplit = (int)std::min<long long>((want + ctas - 1) / ctas, std::max(1, ncols / 64));
    nsplit = std::max(1, std::min(nsplit, 64));
    P.nsplit = nsplit;
    P.partial = nullptr;
    if (nsplit > 1) {
        const int rcs = ensure_plan_scratch(p, (size_t)nsplit * p->nd * p->stride, st);
        if (rcs) return rcs;
        P.partial = p->scratch;
    }
    int rc = CUVDIA_OK;
#define DW_GO(KGV)                                                                                \
    do {                                                                                          \
        const size_t smem = sizeof(float) * 2 * (size_t)BC * (THREADS + PITCH);                   \
        static bool attr[64] = {false};                                                           \
        rc = allow_dynamic_smem(dd2dia_window_kernel<KGV>, smem, attr);                           \
        if (rc) return rc;                                                                        \
        dd2dia_window_kernel<KGV><<<dim3(gx, gy, nsplit), THREADS, smem, st>>>(P);                \
    } while (0)
    if (KG == 32) DW_GO(32); else DW_GO(16);
#undef DW_GO
    count_launch();
    rc = check_launch("dd2dia_window_kernel");
    if (rc) return rc;
    if (nsplit > 1) rc = launch_dd2dia_combine(p, Cv, fa, fc, nsplit, P.partial, st);
    return rc;
}

}  // namespace cuvdia
