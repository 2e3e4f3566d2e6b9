// densedense_to_dia for scattered diagonal patterns (any row factor) whose neighbouring offsets lie
// close enough that a window of the second dense operand fits in shared memory.
//
//   C_dia[k][i] = factC*C_dia[k][i] + factAB * sum_b A[i,b] * B[i/rf + off_k, b]
//
// Every stored cell is a dot product over the batch between a row of A and a row of B; with
// scattered offsets no two cells of a thread share a B row, so B values cannot be reused from
// registers and the ceiling is one shared-memory word per multiply-add (a quarter of the FP32
// rate).  What can be saved is the traffic behind it: the plain kernel fetches every B value from
// L2 once per cell.  Here the diagonals are taken in ascending order of their offsets, 32 (or 16)
// at a time; a block owns 256 rows (512, two per thread, where the row factor divides 256) and one
// such group, and stages, per 8 batch columns, its tile of A and the window of B rows the group can
// touch (rows i/rf + off_min .. off_max of the group; rows outside B arrive as zeros) with 16-byte
// asynchronous copies, one chunk ahead of the arithmetic (two stages).  A staged B value then serves
// every cell of the block on its row - about rows*32/window times - and each thread keeps 32 running
// sums.  Two blocks share an SM, so one block's copies overlap the other's arithmetic.
// The batch is summed in column order within a split and the splits in order by a second kernel,
// so the result does not depend on scheduling.  Only cells inside a diagonal's valid range are
// written (matrix_ops/densedense_to_sparse.cu:104-119).
#include "cuvdia_internal.cuh"

namespace cuvdia {

namespace dw {
constexpr int THREADS = 256;
constexpr int BC = 8;                // batch columns per staged chunk
// words per staged B column for one and two rows per thread: two stages of 41 / 53.5 KB, two blocks per SM
template <int RPT> __host__ __device__ constexpr int pitch() { return RPT == 1 ? 1032 : 1160; }
}

struct DdWindowParams {
    int h, w, nd, S, rf;
    int lda, ldb, ncols, nsplit;
    float fa, fc;
    const float* A; const float* B; float* C; float* partial;
    const int* sorted_slot;          // storage slot of the k-th smallest offset
    const int* sorted_off;           // the k-th smallest offset
};

// KG: diagonals per group (32, or 16 where 32 neighbours span too many rows for the window).  RPT: rows per thread
// (2 where the row factor divides 256, so that the second row's cells sit a constant distance from the first's).
// The pitch of a staged column is a compile-time constant, so that a cell's shared-memory address is a register
// plus an immediate.
template <int KG, int RPT>
__global__ void __launch_bounds__(dw::THREADS, 2)
dd2dia_window_kernel(const DdWindowParams P) {
    using namespace dw;
    constexpr int TR = RPT * THREADS;                // rows per block
    constexpr int PITCH = pitch<RPT>();
    constexpr int STAGE = BC * (TR + PITCH);         // words per stage: A tile [BC][TR], B window [BC][PITCH]
    extern __shared__ __align__(16) float smem[];    // two stages
    const int tid = threadIdx.x;
    const int i0 = blockIdx.x * TR;
    const int g0 = blockIdx.y * KG;                  // first diagonal (in offset order) of the group
    const int gn = min(KG, P.nd - g0);
    const int z = blockIdx.z;
    const int b0 = (int)((long long)P.ncols * z / P.nsplit), b1 = (int)((long long)P.ncols * (z + 1) / P.nsplit);
    const int gmin = P.sorted_off[g0], gmax = P.sorted_off[g0 + gn - 1];
    const int wbase = (i0 / P.rf + gmin) & ~3;       // first staged B row: the window's first row rounded down to 4
    // 16-byte pieces per staged column: the rows a full tile can touch (rows outside B arrive as zeros)
    const int wchunks = ((i0 + TR - 1) / P.rf + gmax - wbase + 4) / 4;
    const int roff = THREADS / P.rf;                 // distance between the cells of a thread's two rows (RPT == 2)

    // word index of the cells of this thread's first row inside stage 0 (indices into the shared array itself, so
    // that the loads below stay in the shared address space)
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

    const unsigned sm_u = (unsigned)__cvta_generic_to_shared(smem);
    // 16-byte asynchronous copies; bytes past the end of an operand (or of this split's columns) arrive as zeros.
    // What does not depend on the chunk is worked out once: this thread's piece of the A tile (in every CPASS-th
    // column) and its pieces of a B column.
    constexpr int PPC = TR / 4;                      // 16-byte pieces per A column
    constexpr int CPASS = THREADS / PPC;             // A columns covered by one pass of the block
    const int qa = tid % PPC, ca = tid / PPC;
    const int rowa = i0 + 4 * qa;
    const unsigned bytes_a = 4u * (unsigned)max(0, min(4, P.h - rowa));
    const float* const srca = P.A + min(rowa, (P.h - 1) & ~3);
    const unsigned dsta = 4u * (unsigned)(ca * TR + 4 * qa);
    auto stage = [&](int buf, int cb) {
        const unsigned base = sm_u + 4u * (unsigned)(buf * STAGE);
#pragma unroll
        for (int u = 0; u < BC / CPASS; u++) {                              // A tile
            const int c = ca + CPASS * u;
            const bool col_ok = cb + c < b1;
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;"
                         ::"r"(base + dsta + 4u * (unsigned)(CPASS * u * TR)),
                           "l"(srca + (size_t)(col_ok ? cb + c : b0) * P.lda), "r"(col_ok ? bytes_a : 0u) : "memory");
        }
        for (int q = tid; q < wchunks; q += THREADS) {                      // B window: piece q of every column
            const int row = wbase + 4 * q;
            const unsigned bytes_b = row >= 0 ? 4u * (unsigned)max(0, min(4, P.w - row)) : 0u;
            const float* const srcb = P.B + min(max(row, 0), (P.w - 1) & ~3);
            const unsigned dstb = base + 4u * (unsigned)(BC * TR + 4 * q);
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
        const float* st2 = st + roff;                // the second row's cells
        // ---- 8 columns x KG cells x RPT rows per thread ----
#pragma unroll
        for (int c = 0; c < BC; c++) {
            const float a0 = st[c * TR + tid];
            const float a1 = RPT == 2 ? st[c * TR + THREADS + tid] : 0.f;
#pragma unroll
            for (int kk = 0; kk < KG; kk++) {
                acc[0][kk] = fmaf(a0, st[cell[kk] + c * PITCH], acc[0][kk]);
                if (RPT == 2) acc[RPT - 1][kk] = fmaf(a1, st2[cell[kk] + c * PITCH], acc[RPT - 1][kk]);
            }
        }
        __syncthreads();                             // everyone is done with this stage before it is refilled
    }

#pragma unroll
    for (int r = 0; r < RPT; r++) {
        const int i = i0 + r * THREADS + tid;
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

int launch_dd2dia_combine(const cuvdia_plan* p, float* Cv, float fa, float fc, int nsplit, const float* partial,
                          cudaStream_t st);

// Rows per thread and diagonals per group for this plan: two rows where the row factor divides 256 and the matrix
// has rows to fill the GPU with such tiles, 32 diagonals if the rows a group can touch fit the staged window, else
// 16; false if nothing fits.
static bool window_shape(const cuvdia_plan* p, int* rpt, int* kg) {
    for (int r = 2; r >= 1; r--) {
        if (r == 2 && (dw::THREADS % p->rf != 0 || p->h < 4 * 2 * dw::THREADS)) continue;
        const int tile = (r * dw::THREADS - 1) / p->rf + 1;
        const int pitch = r == 2 ? dw::pitch<2>() : dw::pitch<1>();
        for (int v = (r == 2 ? 0 : 1); v >= 0; v--)           // two rows x 32 diagonals would not fit the registers
            if (p->group_window_max[v] > 0 && tile + p->group_window_max[v] + 7 <= pitch) {
                *rpt = r; *kg = v == 1 ? 32 : 16;
                return true;
            }
    }
    return false;
}

// Neighbouring diagonals (in offset order) close enough for the window, 16-byte aligned operands, and enough work
// to stage for.
bool dd2dia_window_applicable(const cuvdia_plan* p, const float* A, int lda, const float* B, int ldb, int ncols) {
    auto al16 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
    if (!(al16(A) && al16(B) && lda % 4 == 0 && ldb % 4 == 0)) return false;
    int rpt, kg;
    return p->d_sorted != nullptr && window_shape(p, &rpt, &kg) && p->nd >= 16 && ncols >= 32;
}

int launch_dd2dia_window(cuvdia_plan* p, float* Cv, const float* A, int lda, const float* B, int ldb, int ncols,
                         float fa, float fc, cudaStream_t st) {
    using namespace dw;
    DdWindowParams P;
    P.h = p->h; P.w = p->w; P.nd = p->nd; P.S = p->stride; P.rf = p->rf;
    P.lda = lda; P.ldb = ldb; P.ncols = ncols;
    int RPT = 1, KG = 16;
    if (!window_shape(p, &RPT, &KG)) { set_last_error("window does not fit"); return CUVDIA_ERR_UNSUPPORTED; }
    P.fa = fa; P.fc = fc; P.A = A; P.B = B; P.C = Cv;
    P.sorted_slot = p->d_sorted; P.sorted_off = p->d_sorted + p->nd;
    const int TR = RPT * THREADS;
    const int gx = (p->h + TR - 1) / TR, gy = (p->nd + KG - 1) / KG;
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
#define DW_GO(KGV, RV)                                                                            \
    do {                                                                                          \
        const size_t smem = sizeof(float) * 2 * (size_t)BC * (RV * THREADS + pitch<RV>());        \
        static bool attr[64] = {false};                                                           \
        rc = allow_dynamic_smem(dd2dia_window_kernel<KGV, RV>, smem, attr);                       \
        if (rc) return rc;                                                                        \
        dd2dia_window_kernel<KGV, RV><<<dim3(gx, gy, nsplit), THREADS, smem, st>>>(P);            \
    } while (0)
    if (RPT == 2) DW_GO(16, 2);
    else          { if (KG == 32) DW_GO(32, 1); else DW_GO(16, 1); }
#undef DW_GO
    count_launch();
    rc = check_launch("dd2dia_window_kernel");
    if (rc) return rc;
    if (nsplit > 1) rc = launch_dd2dia_combine(p, Cv, fa, fc, nsplit, P.partial, st);
    return rc;
}

}  // namespace cuvdia
