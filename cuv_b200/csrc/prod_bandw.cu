// prod with a banded DIA operand (consecutive ascending diagonals) whose row factor is larger than 1 (a "steep"
// band: diagonal k holds the cells (i, i/rf + lo + k); the local receptive fields of a layer that shrinks by rf),
// times many batch columns: the band walked as a streaming product.
//
// With offsets lo, lo+1, ..., lo+nd-1 and rf = row_fact (matrix_ops/spmv.cu:161-198)
//     'n':  C[i,b] = sum_k A[k][i] * B[i/rf + lo + k, b]
//     't':  C[j,b] = sum_k sum_{l<rf} A[k][rf*(j-lo-k) + l] * B[rf*(j-lo-k) + l, b]
// (for rf = 1 the register-tiled kernel of prod_band.cu was measured faster - 53.5 against 49.7 TFLOP/s at 1024
// diagonals - and is used instead).  A block owns 32 output rows and 1024 batch columns (512 in the variant
// with 8 rows per thread, which is taken when 512-column tiles waste fewer columns of the batch).  All of its rows walk the SAME dense rows of B,
// X0, X0+1, ... in steps q = 0, 1, ...: output row r of the tile meets B row X0+q on diagonal
// k = q - r/rf - rem ('n') or k = q/rf - (31 - r) - rem ('t'), so one step is the rank-1 update
//     C[r, b] += As[q][r] * B[X0+q, b]
// with the 32 coefficients As[q][.] of the step laid side by side - a product of a [32 x (nd+31)] coefficient
// panel with [(nd+31) x 1024] rows of B, of which each output only uses the nd steps its diagonals cover
// (the other 31 carry zero coefficients: the price of sharing B rows across the tile, 31/nd of the work).
// B is therefore streamed through shared memory exactly once per tile, 16 rows at a time, by TMA tile
// loads (cp.async.bulk.tensor, no multicast, 64-byte swizzle so that the 128-bit reads along a column are
// free of bank conflicts) into a ring of three or four stages; there is no halo and no window to re-load.
// Four producer warps (one of them issues the loads) re-lay ("skew") each slice of the band, as TMA delivers
// it, into the coefficient panel As of the stage, applying factAB and zeroing cells outside the matrix (padding
// cells of the diagonal storage may hold NaN and must never contribute); with a single producer warp the
// consumers waited for coefficients more than they computed (config 1: 259 us, with four 184 us).  Sixteen
// consumer warps (four per scheduler) each own 32 rows x 64 columns, 16 rows x 4 columns per thread: per step
// four 128-bit loads of coefficients (shared by half a warp), a quarter of four 128-bit loads of B, and 32
// packed f32x2 multiply-adds.  Every hand-over is an mbarrier with a bounded,
// warp-uniform wait; consumers never meet a block barrier.
// The transposed product walks the B rows in DESCENDING order (X0 is the highest row the tile needs), so that
// for both products the diagonals an output meets ascend with the step: per output the terms are added in
// diagonal storage order, and the EXACT mode (separate multiply and add) reproduces CUV's host loop
// (matrix_ops/spmv.cu:161-198) bit for bit, except that skipped cells are added as +0 (a -0 accumulator
// becomes +0) and a non-finite B value within a chunk's reach of an output's band meets a zeroed coefficient.
#include <cuda.h>

#include "cuvdia_internal.cuh"

namespace cuvdia {

int make_map_2d_swizzled(CUtensorMap* m, const float* base, long long dim0, long long dim1, long long pitch, int box0,
                         int box1, int swizzle_bytes);

namespace pw {
constexpr int TM = 32;                 // output rows per block
constexpr int NCW = 16;                // consumer warps
constexpr int KC = 16;                 // steps (B rows) per chunk
constexpr int NPW = 4;                 // producer warps (one warp group): one issues the loads, all four re-lay the band slice
constexpr int NRAW = KC + TM - 1;      // diagonals a chunk touches
constexpr int BOXC = 256;              // columns per TMA box of B
constexpr int THREADS = 32 * (NCW + 4);   // warps are allocated four at a time: the producer warp brings three idle ones
// Register budgets after the warp groups re-balance the block's register pool.  The pool is what the block was
// launched with (THREADS x the kernel's register count, REGS_LAUNCH); what the consumers take must have been given
// back by the producer's warp group, or the request would wait for ever.  The host side checks the kernel's actual
// register count against REGS_LAUNCH before it ever launches.
constexpr int REGS_LAUNCH = 96;
constexpr int REGS_CONSUMER = 112;
constexpr int REGS_PRODUCER = 32;
static_assert(NCW * 32 * REGS_CONSUMER + 4 * 32 * REGS_PRODUCER <= THREADS * REGS_LAUNCH,
              "the re-balanced register budgets must fit into the pool the block is launched with");
constexpr int AS_FLOATS = KC * TM;     // one stage of coefficients: [step][32 rows]
constexpr int RAW_FLOATS = NRAW * TM;  // band slice as TMA delivers it ('n': 47 x 32; 't': 47 x 16 uses half)
// RPT = output rows per thread (4 columns each).  16: a warp owns 32 rows x 64 columns, the block 32 x 1024.
// 8: a warp owns 16 rows x 64 columns, two warp rows, the block 32 x 512 - twice the warps for the same outputs,
// for batches that do not fill 1024-column tiles.
template <int RPT> struct Tile {
    static constexpr int WARP_ROWS = TM / (2 * RPT);
    static constexpr int WARP_COLS = NCW / WARP_ROWS;
    static constexpr int TN = 64 * WARP_COLS;              // batch columns per block
    static constexpr int BS_FLOATS = KC * TN;              // one stage of B: [column][16 rows]
    static constexpr int STAGES = RPT == 16 ? 3 : 4;       // 3 x 64 KB or 4 x 32 KB of B in flight
    static constexpr size_t SMEM = sizeof(float) * (STAGES * BS_FLOATS + STAGES * AS_FLOATS + 2 * RAW_FLOATS) + 256;
};
constexpr unsigned SPIN_LIMIT = 1u << 26;
constexpr unsigned DRAIN_LIMIT = 1u << 22;  // second, shorter wait for copies still in flight when a warp gives up
}  // namespace pw

__device__ __forceinline__ unsigned w_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void w_init(unsigned long long* bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(w_u32(bar)), "r"(count));
}
__device__ __forceinline__ void w_expect_tx(unsigned long long* bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(w_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void w_arrive(unsigned long long* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(w_u32(bar)) : "memory");
}
__device__ __forceinline__ bool w_wait(unsigned long long* bar, unsigned parity) {
    const unsigned addr = w_u32(bar);
    for (unsigned it = 0; it < pw::SPIN_LIMIT; it++) {
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
// After a wait has run out: one more bounded wait for a copy this thread issued, so that it does not land in shared
// memory the block has already given back.
__device__ __forceinline__ void w_drain(unsigned long long* bar, unsigned parity) {
    const unsigned addr = w_u32(bar);
    for (unsigned it = 0; it < pw::DRAIN_LIMIT; it++) {
        unsigned done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done) : "r"(addr), "r"(parity) : "memory");
        if (done) return;
    }
}
// warp-uniform: either every lane sees the phase complete or the whole warp gives up
__device__ __forceinline__ bool w_warp_wait(unsigned long long* bar, unsigned parity) {
    return __all_sync(0xffffffffu, w_wait(bar, parity) ? 1 : 0) != 0;
}
__device__ __forceinline__ void w_tma_2d(void* dst, const CUtensorMap* map, int x, int y, unsigned long long* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(w_u32(dst)), "l"(map), "r"(x), "r"(y), "r"(w_u32(bar)) : "memory");
}

template <bool EXACT>
__device__ __forceinline__ void w_mac2(float2& acc, float2 a, float2 b) {
    if (EXACT) {                       // separate roundings: packed multiply, two scalar adds (stays unfused)
        const float2 p = __fmul2_rn(a, b);
        acc.x = __fadd_rn(acc.x, p.x);
        acc.y = __fadd_rn(acc.y, p.y);
    } else {
        acc = __ffma2_rn(a, b, acc);
    }
}

struct BandWParams {
    int h, w, nd, lo, rf;
    int gpc;                  // groups of rf B rows per chunk: KC / rf ('t')
    int rf_shift;             // log2(rf)
    int rows_out, rows_b;     // h, w ('n') or w, h ('t')
    int ncols, ldc;
    int rem;                  // alignment shift (0..3) that keeps every TMA row coordinate a multiple of 4
    int nchunks;
    int last_groups;          // 4-step groups of the last chunk that contain steps of the band (1..4)
    float fa, fc;
    int vec_c;                // C allows 128-bit accesses
    float* C;
    int* status;
};

// Step q of the tile whose first output row is t0 meets B row
//   'n': x = t0/rf + lo - rem + q                       on diagonal k = q - r/rf - rem         for output row t0 + r
//   't': x = rf*(t0 + 31 - lo + rem - q/rf) + q%rf      on diagonal k = q/rf - (31 - r) - rem  for output row t0 + r
// (rem keeps the first row of every 16-row box a multiple of 4, i.e. on a 16-byte boundary).  In both cases the
// diagonals an output meets ascend with q, and for 't' the rf rows of one diagonal's group come in ascending order:
// the order of CUV's host loops.  RFT is the row factor the transposed consumer is compiled for (2, 4 or 8; it
// fixes which element of a 128-bit B vector belongs to which step); 'n' is compiled once (RFT = 1) and takes any
// row factor that divides 8.
template <bool TRANS, bool EXACT, int RFT, int RPT>
__global__ void __launch_bounds__(pw::THREADS, 1)
prod_bandw_kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB,
                  const BandWParams P) {
    using namespace pw;
    constexpr int TN = Tile<RPT>::TN, BS_FLOATS = Tile<RPT>::BS_FLOATS, WARP_COLS = Tile<RPT>::WARP_COLS;
    constexpr int STAGES = Tile<RPT>::STAGES;
    extern __shared__ __align__(1024) float smem_f[];
    float* const Bs0 = smem_f;                                   // [STAGES][TN][KC], swizzled by TMA
    float* const As0 = smem_f + STAGES * BS_FLOATS;              // [STAGES][KC][TM]
    float* const raw0 = As0 + STAGES * AS_FLOATS;                // [2][NRAW x TM]
    unsigned long long* const bars = reinterpret_cast<unsigned long long*>(raw0 + 2 * RAW_FLOATS);
    unsigned long long* const full = bars;                       // [STAGES] B landed (tx) + coefficients written
    unsigned long long* const empty = bars + STAGES;             // [STAGES] one arrival per consumer warp
    unsigned long long* const raw_full = bars + 2 * STAGES;      // [2]
    unsigned long long* const raw_free = bars + 2 * STAGES + 2;  // [2] one arrival per producer warp

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    // column tiles vary fastest across the grid: blocks that run together share the band slice and neighbouring
    // row tiles re-use each other's B rows out of L2
    const int t0 = blockIdx.y * TM;
    const int n0 = blockIdx.x * TN;
    const int nch = P.nchunks;

    if (tid == 0) {
#pragma unroll
        for (int s = 0; s < STAGES; s++) { w_init(&full[s], 1 + NPW); w_init(&empty[s], NCW); }
        w_init(&raw_full[0], 1);
        w_init(&raw_full[1], 1);
        w_init(&raw_free[0], NPW);
        w_init(&raw_free[1], NPW);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    // The kernel is compiled for 96 registers per thread (640 threads: a pool of 61440); the producers' warp group
    // hands back all but 32 per thread and the four consumer warp groups take 112 each (16*32*112 + 4*32*32 = 61440).
    if (warp >= NCW) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(REGS_PRODUCER));
        // =========================== producer warps ===========================
        // Warp pw of the four re-lays steps pw, pw+4, pw+8, pw+12 of every chunk; lane 0 of warp 0 issues the loads.
        const int pw_ = warp - NCW;
        const bool issuer = pw_ == 0 && lane == 0;
        // first B row (TMA x coordinate) and first diagonal (y coordinate) of chunk c
        const int rf = P.rf, rsh = P.rf_shift;               // rf is 1, 2, 4 or 8: divisions become shifts
        auto b_row0 = [&](int c) {
            return TRANS ? rf * (t0 + (TM - 1) - P.lo + P.rem - (c + 1) * P.gpc + 1) : ((t0 >> rsh) + P.lo - P.rem + c * KC);
        };
        auto k0 = [&](int c) { return (TRANS ? c * P.gpc : c * KC) - (TM - 1) - P.rem; };
        constexpr unsigned RAW_TX = sizeof(float) * NRAW * (TRANS ? KC : TM);
        constexpr unsigned BS_TX = sizeof(float) * BS_FLOATS;
        int armed_raw = -1, armed_b = -1;                   // issuer: last chunk whose copies were started
        auto issue_raw = [&](int c) {
            w_expect_tx(&raw_full[c & 1], RAW_TX);
            // 'n': the tile's 32 rows of each diagonal;  't': the chunk's 16 matrix rows (= its B rows) of each diagonal
            w_tma_2d(raw0 + (c & 1) * RAW_FLOATS, &mapA, TRANS ? b_row0(c) : t0, k0(c), &raw_full[c & 1]);
            armed_raw = c;
        };
        // a producer that gives up: the issuing thread first waits, bounded again, for the copies it started (the
        // band slices of the last two chunks and the B stages of the last STAGES chunks)
        auto give_up = [&]() {
            if (lane == 0 && P.status) *P.status = 3;
            if (issuer) {
                for (int c2 = max(0, armed_raw - 1); c2 <= armed_raw; c2++) w_drain(&raw_full[c2 & 1], (c2 >> 1) & 1);
                for (int c2 = max(0, armed_b - STAGES + 1); c2 <= armed_b; c2++) w_drain(&full[c2 % STAGES], (c2 / STAGES) & 1);
            }
        };
        if (issuer) { issue_raw(0); if (nch > 1) issue_raw(1); }
        for (int c = 0; c < nch; c++) {
            const int s = c % STAGES;
            bool ok = true;
            if (c >= STAGES) ok = w_warp_wait(&empty[s], ((c / STAGES) - 1) & 1);
            if (!ok) { give_up(); return; }
            if (issuer) {
                armed_b = c;
                w_expect_tx(&full[s], BS_TX);
#pragma unroll
                for (int bx = 0; bx < TN / BOXC; bx++)
                    w_tma_2d(Bs0 + s * BS_FLOATS + bx * (KC * BOXC), &mapB, b_row0(c), n0 + bx * BOXC, &full[s]);
            }
            ok = w_warp_wait(&raw_full[c & 1], (c >> 1) & 1);
            if (!ok) { give_up(); return; }
            // ---- skew: As[qq][r] = factAB * A[k][matrix row] for the diagonal k that output row r meets at step qq, zero
            // where the cell lies outside the matrix.  Lane = output row r of the tile.
            //   'n': k = k0 + 31 + qq - r/rf,  slice [diagonal][32 tile rows]
            //   't': k = k0 + qq/rf + r,       slice [diagonal][16 B rows]; step qq reads box row rf*(gpc-1-qq/rf) + qq%rf
            // For 't' every lane starts at a different step (qq rotated by the lane), so that the 32 reads of one
            // instruction fall into 16 different banks instead of 2. ----
            const float* raw = raw0 + (c & 1) * RAW_FLOATS;
            float* as = As0 + s * AS_FLOATS;
            const int kc0 = k0(c), xb = b_row0(c);
            // chunk-uniform: every cell the chunk touches lies inside the matrix ('t': whole groups of rf rows)
            const bool interior = kc0 >= 0 && kc0 + NRAW <= P.nd && xb >= 0 && xb + KC <= P.rows_b &&
                                  (TRANS || t0 + TM <= P.h);
            const int rdiv = lane >> rsh;
#pragma unroll
            for (int it = 0; it < KC / NPW; it++) {
                const int qq = TRANS ? ((pw_ + NPW * it + lane) & (KC - 1)) : pw_ + NPW * it;
                const int gq = qq >> rsh;                             // 't': group of rf rows within the chunk
                const int brow = TRANS ? rf * (P.gpc - 1 - gq) + (qq - (gq << rsh)) : qq;  // row of the B box this step reads
                const int kk = TRANS ? gq + lane : qq - rdiv + (TM - 1);                  // row of the slice: diagonal kc0 + kk
                float v = TRANS ? raw[kk * KC + brow] : raw[kk * TM + lane];
                if (!interior || P.fa != 1.f) {
                    const int k = kc0 + kk;
                    const int x = xb + brow;                                             // B row of the step
                    bool in = (unsigned)k < (unsigned)P.nd;
                    // 'n': cell (t0 + r, x): row and column must exist;  't': cell (x, t0 + r): the whole group of rf
                    // rows must lie inside the matrix (matrix_ops/spmv.cu:168: N counts whole groups only)
                    if (!TRANS) in = in && (unsigned)x < (unsigned)P.w && t0 + lane < P.h;
                    else { const int m = x >= 0 ? (x >> rsh) : -1; in = in && m >= 0 && (long long)(m + 1) * rf <= P.h; }
                    if (P.fa != 1.f) v = __fmul_rn(P.fa, v);
                    v = in ? v : 0.f;
                }
                as[qq * TM + lane] = v;
            }
            __syncwarp();
            if (lane == 0) { w_arrive(&full[s]); w_arrive(&raw_free[c & 1]); }
            // the slice buffer may be refilled once all four warps have read it (a bounded wait, like every other)
            if (issuer && c + 2 < nch) {
                if (!w_wait(&raw_free[c & 1], (c >> 1) & 1)) { if (P.status) *P.status = 3; }
                else issue_raw(c + 2);
            }
            __syncwarp();
        }
        return;
    }

    // =========================== consumer warps ===========================
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(REGS_CONSUMER));
    const int rg = lane >> 4, cg = lane & 15;
    const int wr = warp / WARP_COLS, wc = warp % WARP_COLS;
    // this thread: rows t0 + row0 .. + RPT-1, columns n0 + 64*wc + cg + 16*cc (cc = 0..3)
    const int row0 = (2 * wr + rg) * RPT;
    const int colb = 64 * wc + cg;
    const int sw = (cg >> 1) & 3;                 // 64-byte swizzle: 16-byte chunk j of column c sits at j ^ ((c >> 1) & 3)

    float2 acc[RPT / 2][4];                       // acc[jp][cc]: rows (2jp, 2jp+1) of column cc
#pragma unroll
    for (int jp = 0; jp < RPT / 2; jp++)
#pragma unroll
        for (int cc = 0; cc < 4; cc++) acc[jp][cc] = make_float2(0.f, 0.f);
    if (P.fc != 0.f) {
#pragma unroll
        for (int cc = 0; cc < 4; cc++) {
            const int col = n0 + colb + 16 * cc;
#pragma unroll
            for (int j = 0; j < RPT; j++) {
                const int row = t0 + row0 + j;
                if (col < P.ncols && row < P.rows_out) {
                    const float v = __fmul_rn(P.C[(size_t)col * P.ldc + row], P.fc);
                    if (j & 1) acc[j >> 1][cc].y = v; else acc[j >> 1][cc].x = v;
                }
            }
        }
    }

    // 16-byte chunk of a column's 16 rows that the steps of group g read: 'n' ascending; 't' the groups of RFT rows
    // descend through the box (RFT 8: two chunks per group, ascending inside it)
    auto bchunk = [](int g) { return !TRANS ? g : RFT == 8 ? ((g & 2) ^ 2) + (g & 1) : 3 - g; };
    // a warp whose 64 columns all lie beyond the batch keeps the hand-over going and leaves the arithmetic out
    const bool has_columns = n0 + 64 * wc < P.ncols;
    for (int c = 0; c < nch; c++) {
        const int s = c % STAGES;
        if (!w_warp_wait(&full[s], (c / STAGES) & 1)) { if (lane == 0 && P.status) *P.status = 3; return; }
        if (!has_columns) { if (lane == 0) w_arrive(&empty[s]); continue; }
        const float* bsp = Bs0 + s * BS_FLOATS + colb * KC;
        const float* asp = As0 + s * AS_FLOATS + row0;
        const int ng = c == nch - 1 ? P.last_groups : KC / 4;
#pragma unroll
        for (int g = 0; g < KC / 4; g++) {
            if (g < ng) {
                float4 bw[4];
#pragma unroll
                for (int cc = 0; cc < 4; cc++)
                    bw[cc] = *reinterpret_cast<const float4*>(bsp + cc * 16 * KC + ((bchunk(g) ^ sw) << 2));
#pragma unroll
                for (int u = 0; u < 4; u++) {
                    const float* ap = asp + (4 * g + u) * TM;
                    float2 a[RPT / 2];
#pragma unroll
                    for (int v = 0; v < RPT / 4; v++) {
                        const float4 av = *reinterpret_cast<const float4*>(ap + 4 * v);
                        a[2 * v] = make_float2(av.x, av.y);
                        a[2 * v + 1] = make_float2(av.z, av.w);
                    }
#pragma unroll
                    for (int cc = 0; cc < 4; cc++) {
                        // which element of the vector step u reads: 'n' ascending; 't' groups of RFT rows descending,
                        // ascending inside a group (RFT 2: z w x y, RFT 4 and 8: x y z w)
                        const int e = (TRANS && RFT == 2) ? (u ^ 2) : u;
                        const float b = e == 0 ? bw[cc].x : e == 1 ? bw[cc].y : e == 2 ? bw[cc].z : bw[cc].w;
                        const float2 bb = make_float2(b, b);
#pragma unroll
                        for (int jp = 0; jp < RPT / 2; jp++) w_mac2<EXACT>(acc[jp][cc], a[jp], bb);
                    }
                }
            }
        }
        __syncwarp();
        if (lane == 0) w_arrive(&empty[s]);
    }

    // ---- store ----
#pragma unroll
    for (int cc = 0; cc < 4; cc++) {
        const int col = n0 + colb + 16 * cc;
        if (col >= P.ncols) continue;
        const int orow = t0 + row0;
        float* cp = P.C + (size_t)col * P.ldc + orow;
        if (P.vec_c && orow + RPT <= P.rows_out) {
#pragma unroll
            for (int v = 0; v < RPT / 4; v++)
                *reinterpret_cast<float4*>(cp + 4 * v) =
                    make_float4(acc[2 * v][cc].x, acc[2 * v][cc].y, acc[2 * v + 1][cc].x, acc[2 * v + 1][cc].y);
        } else {
#pragma unroll
            for (int j = 0; j < RPT; j++)
                if (orow + j < P.rows_out) cp[j] = (j & 1) ? acc[j >> 1][cc].y : acc[j >> 1][cc].x;
        }
    }
}

// ---- host side ----------------------------------------------------------------------------------------

static inline bool w_al16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// The register re-balancing inside the kernel is only safe if every instantiation was compiled with exactly the
// register count its budgets were derived from (a smaller pool would leave the consumers waiting for registers).
template <bool TRANS, bool EXACT, int RFT>
static bool bandw_pool_ok_one() {
    cudaFuncAttributes a, b;
    return cudaFuncGetAttributes(&a, prod_bandw_kernel<TRANS, EXACT, RFT, 16>) == cudaSuccess && a.numRegs == pw::REGS_LAUNCH &&
           cudaFuncGetAttributes(&b, prod_bandw_kernel<TRANS, EXACT, RFT, 8>) == cudaSuccess && b.numRegs == pw::REGS_LAUNCH;
}
static bool bandw_register_pool_ok() {
    static int cached = -1;
    if (cached < 0) {
        const bool ok = bandw_pool_ok_one<false, false, 1>() && bandw_pool_ok_one<false, true, 1>() &&
                        bandw_pool_ok_one<true, false, 2>() && bandw_pool_ok_one<true, true, 2>() &&
                        bandw_pool_ok_one<true, false, 4>() && bandw_pool_ok_one<true, true, 4>() &&
                        bandw_pool_ok_one<true, false, 8>() && bandw_pool_ok_one<true, true, 8>();
        cached = ok ? 1 : 0;
    }
    return cached == 1;
}

bool prod_bandw_applicable(const cuvdia_plan* p, const float* A, const float* B, int ldb, int ncols) {
    // Row factors 2, 4, 8 (a chunk of 16 B rows must hold whole groups of rf rows, and the first B row of a tile,
    // t0/rf, must stay a multiple of 4); enough diagonals to pay for the up to 31 extra steps of a tile; and enough
    // batch columns to keep at least four of the sixteen consumer warps busy.
    if (!(p->rf == 2 || p->rf == 4 || p->rf == 8)) return false;
    if (p->nd < 32 || ncols < 256) return false;
    return p->is_band && w_al16(A) && w_al16(B) && p->stride % 4 == 0 && ldb % 4 == 0 && tma_available() &&
           bandw_register_pool_ok();
}

template <bool TRANS, bool EXACT, int RFT, int RPT>
static int launch_bandw_t(const cuvdia_plan* p, const float* A, const float* B, int ldb, float* C, int ldc, int ncols,
                          float fa, float fc, cudaStream_t st) {
    using namespace pw;
    constexpr int TN = Tile<RPT>::TN;
    constexpr size_t SMEM = Tile<RPT>::SMEM;
    CUtensorMap mapA, mapB;
    int rc = make_map_2d_swizzled(&mapA, A, p->h, p->nd, p->stride, TRANS ? KC : TM, NRAW, 0);
    if (rc) return rc;
    rc = make_map_2d_swizzled(&mapB, B, TRANS ? p->h : p->w, ncols, ldb, KC, BOXC, 64);
    if (rc) return rc;
    BandWParams P;
    P.h = p->h; P.w = p->w; P.nd = p->nd; P.lo = p->band_lo; P.rf = p->rf;
    P.gpc = KC / p->rf;
    P.rf_shift = p->rf == 8 ? 3 : p->rf == 4 ? 2 : p->rf == 2 ? 1 : 0;
    P.rows_out = TRANS ? p->w : p->h;
    P.rows_b = TRANS ? p->h : p->w;
    P.ncols = ncols; P.ldc = ldc;
    // the first B row of a chunk must be a multiple of 4:  'n': t0/rf + lo - rem + 16c;  't': rf*(t0 + 32 - lo + rem) - 16(c+1)
    const int g = TRANS ? (p->rf >= 4 ? 1 : 2) : 4;
    P.rem = ((p->band_lo % g) + g) % g;
    const int steps = TRANS ? p->rf * (p->nd + (TM - 1) + P.rem) : p->nd + (TM - 1) / p->rf + P.rem;
    P.nchunks = (steps + KC - 1) / KC;
    P.last_groups = (steps - (P.nchunks - 1) * KC + 3) / 4;
    P.fa = fa; P.fc = fc;
    P.vec_c = (w_al16(C) && ldc % 4 == 0) ? 1 : 0;
    P.C = C; P.status = p->d_status;
    static bool attr_done[64] = {false};          // one flag set per template instantiation
    rc = allow_dynamic_smem(prod_bandw_kernel<TRANS, EXACT, RFT, RPT>, SMEM, attr_done);
    if (rc) return rc;
    const int gx = (P.rows_out + TM - 1) / TM, gy = (ncols + TN - 1) / TN;
    if (gx > 65535) { set_last_error("too many rows for the banded kernel"); return CUVDIA_ERR_UNSUPPORTED; }
    prod_bandw_kernel<TRANS, EXACT, RFT, RPT><<<dim3(gy, gx), THREADS, SMEM, st>>>(mapA, mapB, P);
    count_launch();
    return check_launch("prod_bandw_kernel");
}

int launch_prod_bandw(const cuvdia_plan* p, const float* A, const float* B, int ldb, float* C, int ldc, int ncols,
                      bool trans, float fa, float fc, int mode, cudaStream_t st) {
    const bool exact = mode == CUVDIA_MODE_EXACT;
    // 512-column tiles (8 rows per thread, twice the warps) when they waste fewer columns than 1024-column tiles
    const bool narrow = (ncols + 511) / 512 * 512 < (ncols + 1023) / 1024 * 1024;
#define GO(TR, RFT)                                                                                              \
    do {                                                                                                         \
        if (narrow) return exact ? launch_bandw_t<TR, true, RFT, 8>(p, A, B, ldb, C, ldc, ncols, fa, fc, st)     \
                                 : launch_bandw_t<TR, false, RFT, 8>(p, A, B, ldb, C, ldc, ncols, fa, fc, st);   \
        return exact ? launch_bandw_t<TR, true, RFT, 16>(p, A, B, ldb, C, ldc, ncols, fa, fc, st)                \
                     : launch_bandw_t<TR, false, RFT, 16>(p, A, B, ldb, C, ldc, ncols, fa, fc, st);              \
    } while (0)
    if (!trans) GO(false, 1);
    if (p->rf == 2) GO(true, 2);
    if (p->rf == 4) GO(true, 4);
    GO(true, 8);
#undef GO
}

}  // namespace cuvdia
