// densedense_to_dia for a banded pattern (consecutive ascending diagonals; row_fact 1, or a power of two up
// to 32 - a "steep" band, the local receptive fields of a layer that shrinks by row_fact).
//
//   G[k][i] = factC*G[k][i] + factAB * sum_b A[i,b] * B[i/rf+lo+k, b],   k = 0..nd-1
//
// is the product A*B^T restricted to a band, so it is computed as dense 128 x 128 tiles of A*B^T
// that cover the band: block (ti, t, z) owns rows i0 = 128*ti of A, rows j0 = i0/rf + lo - rem + 128*t
// of B and the z-th share of the batch.  Both operands are column-major, so a tile of 128 rows x 32
// batch columns is one TMA box (cp.async.bulk.tensor, no multicast) and lands in shared memory as
// [batch column][row]: exactly the layout an outer-product inner loop wants - per batch column a
// thread reads 8 values of each operand with four 128-bit loads and issues 32 packed fused
// multiply-adds (f32x2) into its 8 x 8 accumulators.  Three stages are kept in flight and two blocks
// share an SM.  Rows/columns outside the operands arrive as zeros.  At the end every accumulator
// that lies on a stored diagonal inside the matrix is written to its DIA cell (cells outside the
// diagonals' ranges are never touched, matrix_ops/densedense_to_sparse.cu:104-119); with a batch
// split the partial tiles go to plan-owned scratch and dd2dia_combine_kernel adds them in split
// order.  The two triangular end tiles of each row block compute products the band does not need -
// the price of the dense formulation (128/nd of the work); the quadrant of an end tile that lies
// entirely outside the band is left out, which takes a quarter off that price.
#include <cuda.h>

#include "cuvdia_internal.cuh"

namespace cuvdia {

int make_map_2d(CUtensorMap* m, const float* base, long long dim0, long long dim1, long long pitch, int box0, int box1);
__global__ void dd2dia_combine_kernel(float* __restrict__ Cv, const int* __restrict__ offs, int nd, int h, int w,
                                      int S, int rf, float fa, float fc, int nsplit,
                                      const float* __restrict__ partial);

namespace db {
// 32 batch columns per stage and 3 stages were the best of the (16, 32, 64) x (2, 3, 4) combinations that fit
constexpr int TI = 128, TJ = 128, KB = 32, STAGES = 3, THREADS = 256;
constexpr int TILE_FLOATS = TI * KB;                 // one operand tile of one stage
constexpr size_t SMEM = sizeof(float) * 2 * TILE_FLOATS * STAGES + 128;
constexpr unsigned SPIN_LIMIT = 1u << 26;
}  // namespace db

__device__ __forceinline__ unsigned dsmem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ bool dmbar_wait(unsigned long long* bar, unsigned parity) {
    const unsigned addr = dsmem_u32(bar);
    for (unsigned it = 0; it < db::SPIN_LIMIT; it++) {
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

__device__ __forceinline__ void dmbar_wait_short(unsigned long long* bar, unsigned parity) {
    const unsigned addr = dsmem_u32(bar);
    for (unsigned it = 0; it < (1u << 22); it++) {
        unsigned done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done) : "r"(addr), "r"(parity) : "memory");
        if (done) return;
    }
}

struct DdBandParams {
    int h, w, nd, lo, S, ncols;
    int rf, rf_shift;   // row factor (a power of two) and its logarithm
    int rem;            // lo mod 4 (non-negative): keeps the TMA row coordinate of B 16-byte aligned
    int nsplit;
    int tile0, ntiles;  // this launch covers column tiles tile0 .. tile0 + gridDim.x - 1 of the ntiles of a row block
    float fa, fc;
    float* G;
    float* partial;     // [nsplit][nd*S] when nsplit > 1
    int* status;
};

// One stage: 32 batch columns of the 8 x 8 outer product of a thread.  SKIP names a quadrant of the tile that lies
// entirely outside the band and is left out (block-uniform): 1 = rows 64.. x columns ..63 (the first tile of a
// row block, below the first diagonal), 2 = rows ..63 x columns 64.. (the last tile, above the last diagonal),
// 3 = everything but rows 64.. x columns ..63 (a last tile that the band only touches in that corner).
template <int SKIP>
__device__ __forceinline__ void dd_band_stage(const float* xs, const float* hs, float2 (&acc)[8][4]) {
    using namespace db;
#pragma unroll 8
    for (int b = 0; b < KB; b++) {
        const float4 x0 = *reinterpret_cast<const float4*>(xs + b * TI);
        const float4 x1 = *reinterpret_cast<const float4*>(xs + b * TI + 64);
        const float4 h0 = *reinterpret_cast<const float4*>(hs + b * TJ);
        const float4 h1 = *reinterpret_cast<const float4*>(hs + b * TJ + 64);
        const float x[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
        const float2 hp[4] = {make_float2(h0.x, h0.y), make_float2(h0.z, h0.w), make_float2(h1.x, h1.y),
                              make_float2(h1.z, h1.w)};
#pragma unroll
        for (int ii = 0; ii < 8; ii++) {
            const float2 xx = make_float2(x[ii], x[ii]);
#pragma unroll
            for (int jp = 0; jp < 4; jp++) {
                if (SKIP == 1 && ii >= 4 && jp < 2) continue;
                if (SKIP == 2 && ii < 4 && jp >= 2) continue;
                if (SKIP == 3 && !(ii >= 4 && jp < 2)) continue;
                acc[ii][jp] = __ffma2_rn(xx, hp[jp], acc[ii][jp]);
            }
        }
    }
}

__global__ void __launch_bounds__(db::THREADS, 2)
dd2dia_band_kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB,
                   const DdBandParams P) {
    using namespace db;
    extern __shared__ __align__(1024) float smem_f[];
    float* const Xs0 = smem_f;                                  // [STAGES][KB][TI]
    float* const Hs0 = smem_f + STAGES * TILE_FLOATS;           // [STAGES][KB][TJ]
    unsigned long long* const full = reinterpret_cast<unsigned long long*>(smem_f + 2 * STAGES * TILE_FLOATS);
    unsigned long long* const empty = full + STAGES;      // one arrival per warp when it is done with a stage

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int R = warp * 2 + (lane >> 4);        // row group 0..15: rows 4R..4R+3 and 64+4R..64+4R+3 of the tile
    const int cg = lane & 15;                    // column group: columns 4cg..4cg+3 and 64+4cg..64+4cg+3
    // the column tiles of one row block are neighbours in the grid: they share the A tile, and
    // adjacent row blocks share most B tiles, so both operands come from HBM about once
    const int i0 = blockIdx.y * TI;
    const int tile = P.tile0 + (int)blockIdx.x;
    const int j0 = (i0 >> P.rf_shift) + P.lo - P.rem + tile * TJ;
    const int z = blockIdx.z;
    const int nch_all = (P.ncols + KB - 1) / KB;
    const int ch0 = (int)((long long)nch_all * z / P.nsplit), ch1 = (int)((long long)nch_all * (z + 1) / P.nsplit);
    const int nch = ch1 - ch0;

    // A cell (row ir, column jc of the tile) is on a stored diagonal iff 0 <= jc - ir - rem + 128*t < nd.  In the
    // first tile of a row block the quadrant rows 64.. x columns ..63 never is; in the last one the quadrant
    // rows ..63 x columns 64.. is not either when the band ends at or before the tile's main diagonal, and when it
    // ends 63 or more diagonals before it only the quadrant rows 64.. x columns ..63 is left.
    const int dlast = P.nd + P.rem - TJ * tile;                   // cells of this tile need jc - ir < dlast
    // (with a row factor the band crosses a tile at another slope: no quadrant is left out)
    const int skip = P.rf != 1 ? 0 : tile == 0 ? 1 : (tile == P.ntiles - 1 && dlast <= 1) ? (dlast <= -63 ? 3 : 2) : 0;

    constexpr unsigned TX_BYTES = sizeof(float) * 2 * TILE_FLOATS;
    auto issue = [&](int c) {
        const int s = c % STAGES;
        const unsigned bar = dsmem_u32(&full[s]);
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(TX_BYTES) : "memory");
        asm volatile(
            "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
            ::"r"(dsmem_u32(Xs0 + s * TILE_FLOATS)), "l"(&mapA), "r"(i0), "r"((ch0 + c) * KB), "r"(bar) : "memory");
        asm volatile(
            "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
            ::"r"(dsmem_u32(Hs0 + s * TILE_FLOATS)), "l"(&mapB), "r"(j0), "r"((ch0 + c) * KB), "r"(bar) : "memory");
    };

    if (tid == 0) {
#pragma unroll
        for (int s = 0; s < STAGES; s++) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(dsmem_u32(&full[s])));
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(dsmem_u32(&empty[s])), "r"(THREADS / 32));
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (tid == 0)
        for (int c = 0; c < STAGES && c < nch; c++) issue(c);

    // acc[ii][jp]: row ii of the thread's 8, columns (2jp, 2jp+1) as a packed pair
    float2 acc[8][4];
#pragma unroll
    for (int ii = 0; ii < 8; ii++)
#pragma unroll
        for (int jp = 0; jp < 4; jp++) acc[ii][jp] = make_float2(0.f, 0.f);

    for (int c = 0; c < nch; c++) {
        const int s = c % STAGES;
        if (!dmbar_wait(&full[s], (c / STAGES) & 1)) {
            if (P.status) *P.status = 2;
            // the issuing thread waits once more, bounded, for the copies it started (this chunk's and the ones ahead
            // of it), so that none lands in shared memory the block has given back
            if (tid == 0)
                for (int c2 = c; c2 < nch && c2 < c + STAGES; c2++) dmbar_wait_short(&full[c2 % STAGES], (c2 / STAGES) & 1);
            return;
        }
        const float* xs = Xs0 + s * TILE_FLOATS + 4 * R;
        const float* hs = Hs0 + s * TILE_FLOATS + 4 * cg;
        if (skip == 0) dd_band_stage<0>(xs, hs, acc);
        else if (skip == 1) dd_band_stage<1>(xs, hs, acc);
        else if (skip == 2) dd_band_stage<2>(xs, hs, acc);
        else dd_band_stage<3>(xs, hs, acc);
        // hand the stage back: one arrival per warp; only the issuing thread waits for all of them, so the
        // other warps run ahead into the stages that are already loaded instead of meeting a block barrier
        __syncwarp();
        if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(dsmem_u32(&empty[s])) : "memory");
        if (tid == 0 && c + STAGES < nch) {
            if (!dmbar_wait(&empty[s], (c / STAGES) & 1)) { if (P.status) *P.status = 2; }
            else issue(c + STAGES);
        }
        __syncwarp();
    }

    // ---- write the accumulators that lie on stored diagonals inside the matrix ----
    float* out = P.nsplit == 1 ? P.G : P.partial + (size_t)z * P.nd * P.S;
#pragma unroll
    for (int ii = 0; ii < 8; ii++) {
        const int i = i0 + 4 * R + (ii & 3) + (ii >> 2) * 64;
        if (i >= P.h) continue;
#pragma unroll
        for (int jj = 0; jj < 8; jj++) {
            const int j = j0 + 4 * cg + (jj & 3) + (jj >> 2) * 64;
            const int k = j - (i >> P.rf_shift) - P.lo;
            if ((unsigned)k >= (unsigned)P.nd || (unsigned)j >= (unsigned)P.w) continue;
            const float v = (jj & 1) ? acc[ii][jj >> 1].y : acc[ii][jj >> 1].x;
            float* cell = out + (size_t)k * P.S + i;
            if (P.nsplit == 1) {
                float sv = v;
                if (P.fa != 1.f) sv = __fmul_rn(P.fa, sv);
                *cell = (P.fc != 0.f) ? __fadd_rn(__fmul_rn(P.fc, *cell), sv) : sv;
            } else {
                *cell = v;
            }
        }
    }
}

static inline bool al16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

static int band_tiles(const cuvdia_plan* p);

// Row factor 1, or a power of two up to 32 (a tile's first B row, i0 / rf, must stay a multiple of 4) when the dense
// tiles are at least three tenths band: the staged-window kernel, which the steep band would otherwise take, runs at
// a quarter of the FP32 rate but computes nothing beside the band.
bool dd2dia_band_applicable(const cuvdia_plan* p, const float* A, int lda, const float* B, int ldb, int ncols) {
    if (!(p->is_band && al16(A) && al16(B) && lda % 4 == 0 && ldb % 4 == 0 && ncols >= 1 && p->nd >= 16 && tma_available()))
        return false;
    if (p->rf == 1) return true;
    if (!(p->rf == 2 || p->rf == 4 || p->rf == 8 || p->rf == 16 || p->rf == 32)) return false;
    return 10LL * p->nd >= 3LL * db::TJ * band_tiles(p) && ncols >= 64;
}

// Column tiles per row block, and how a call may be cut in two launches so that the diagonals' array is finished
// slab by slab: tile t writes diagonals 128t - rem - 127 .. 128t - rem + 127, so after tiles 0 .. T-1 the diagonals
// 0 .. 128(T-1) - rem are complete (they are contiguous in memory: a band is stored in ascending order).
static int band_tiles(const cuvdia_plan* p) {
    const int rem = ((p->band_lo % 4) + 4) % 4;
    // the rows of B a block of 128 rows of A touches: rem + (0 .. 127) / rf + (0 .. nd-1)
    return (p->nd + (db::TI - 1) / p->rf + rem + db::TJ - 1) / db::TJ;
}

// Finds a cut T (tiles 0..T-1, then T..gy-1) that needs no more waves of blocks than the uncut grid and finishes as
// close to half of the diagonals as possible with its first launch; 0 if the call should stay one launch (batch split
// in use, too few tiles, or every cut costs a wave; with `force` the waves are not looked at and two tiles are enough).
// *first_diagonals = diagonals complete after the first launch.
int dd2dia_band_cut(const cuvdia_plan* p, int ncols, int* first_diagonals, bool force) {
    const int rem = ((p->band_lo % 4) + 4) % 4;
    const int gx = (p->h + db::TI - 1) / db::TI, gy = band_tiles(p);
    const long long slots = 2LL * sm_count();
    auto waves = [&](long long ctas) { return (ctas + slots - 1) / slots; };
    if (gy < (force ? 3 : 4) || p->rf != 1) return 0;
    int best = 0, best_dist = 1 << 30;
    for (int T = 2; T < gy; T++) {
        if (!force && waves((long long)gx * T) + waves((long long)gx * (gy - T)) > waves((long long)gx * gy)) continue;
        const int done = db::TJ * (T - 1) - rem + 1;
        if (done <= 0) continue;
        const int dist = abs(2 * done - p->nd);
        if (dist < best_dist) { best_dist = dist; best = T; *first_diagonals = std::min(done, p->nd); }
    }
    (void)ncols;
    return best;
}

static int launch_dd2dia_band_tiles(cuvdia_plan* p, float* Cv, const float* A, int lda, const float* B, int ldb, int ncols,
                                    float fa, float fc, int tile0, int tile1, int nsplit, cudaStream_t st);

int launch_dd2dia_band(cuvdia_plan* p, float* Cv, const float* A, int lda, const float* B, int ldb, int ncols,
                       float fa, float fc, cudaStream_t st) {
    return launch_dd2dia_band_tiles(p, Cv, A, lda, B, ldb, ncols, fa, fc, 0, -1, 0, st);
}

// The batch split a whole call would use (1 = none).  A split costs a pass over its partial sums by a second kernel
// and shortens every block's pipeline, while a last wave that is only partly filled costs less than it seems (a block
// alone on an SM runs nearly twice as fast): measured at 16384 rows x 512 diagonals x 1024 columns, 640 tiles,
// 0.381 ms unsplit against 0.454 / 0.473 / 0.512 ms with 2 / 3 / 5 shares.  So the batch is split only when the tiles
// do not fill the GPU once, and then just far enough that they do.
int dd2dia_band_nsplit(const cuvdia_plan* p, int ncols) {
    using namespace db;
    const long long gx = (p->h + TI - 1) / TI, gy = band_tiles(p);
    const long long slots = 2LL * sm_count(), ctas = gx * gy;
    const int nch_all = (ncols + KB - 1) / KB;
    if (ctas >= slots) return 1;
    const long long want = (slots + ctas - 1) / ctas;
    return (int)std::max<long long>(1, std::min<long long>(std::min<long long>(want, 8), std::max(1, nch_all / 4)));
}

// Column tiles tile0 .. tile1-1 (tile1 < 0: all) of every row block; force_nsplit > 0 overrides the batch split.
int launch_dd2dia_band_range(cuvdia_plan* p, float* Cv, const float* A, int lda, const float* B, int ldb, int ncols,
                             float fa, float fc, int tile0, int tile1, cudaStream_t st) {
    return launch_dd2dia_band_tiles(p, Cv, A, lda, B, ldb, ncols, fa, fc, tile0, tile1, 1, st);
}

static int launch_dd2dia_band_tiles(cuvdia_plan* p, float* Cv, const float* A, int lda, const float* B, int ldb, int ncols,
                                    float fa, float fc, int tile0, int tile1, int force_nsplit, cudaStream_t st) {
    using namespace db;
    CUtensorMap mapA, mapB;
    int rc = make_map_2d(&mapA, A, p->h, ncols, lda, TI, KB);
    if (rc) return rc;
    rc = make_map_2d(&mapB, B, p->w, ncols, ldb, TJ, KB);
    if (rc) return rc;
    DdBandParams P;
    P.h = p->h; P.w = p->w; P.nd = p->nd; P.lo = p->band_lo; P.S = p->stride; P.ncols = ncols;
    P.rem = ((p->band_lo % 4) + 4) % 4;
    P.rf = p->rf; P.rf_shift = 0;
    while ((1 << P.rf_shift) < p->rf) P.rf_shift++;
    P.fa = fa; P.fc = fc; P.G = Cv; P.status = p->d_status;
    const int gx = (p->h + TI - 1) / TI;
    const int gy = band_tiles(p);                                // column tiles that cover the band of one row block
    if (tile1 < 0) tile1 = gy;
    // split the batch when the tiles alone leave SMs idle or quantise badly into waves
    const int nsplit = force_nsplit > 0 ? force_nsplit : dd2dia_band_nsplit(p, ncols);
    P.nsplit = nsplit;
    P.tile0 = tile0; P.ntiles = gy;
    P.partial = nullptr;
    if (nsplit > 1) {
        rc = ensure_plan_scratch(p, (size_t)nsplit * p->nd * p->stride, st);
        if (rc) return rc;
        P.partial = p->scratch;
    }
    static bool attr_done[64] = {false};
    rc = allow_dynamic_smem(dd2dia_band_kernel, SMEM, attr_done);
    if (rc) return rc;
    if (gx > 65535 || nsplit > 65535) { set_last_error("matrix too tall for the banded densedense_to_dia"); return CUVDIA_ERR_UNSUPPORTED; }
    dd2dia_band_kernel<<<dim3(tile1 - tile0, gx, nsplit), THREADS, SMEM, st>>>(mapA, mapB, P);
    count_launch();
    rc = check_launch("dd2dia_band_kernel");
    if (rc) return rc;
    if (nsplit > 1) {
        dim3 g2((p->h + 255) / 256, std::min(p->nd, 65535));
        dd2dia_combine_kernel<<<g2, 256, 0, st>>>(Cv, p->d_offsets, p->nd, p->h, p->w, p->stride, p->rf, fa, fc,
                                                  nsplit, P.partial);
        count_launch();
        rc = check_launch("dd2dia_combine_kernel");
    }
    return rc;
}

}  // namespace cuvdia
