// prod with a banded DIA operand (consecutive ascending diagonals, row_fact 1): the tiled kernel.
//
// With offsets lo, lo+1, ..., lo+nd-1 the product is a 1-D stencil with spatially varying
// coefficients,   'n':  C[i,b] = sum_k A[k][i]       * B[i+lo+k, b]
//                 't':  C[j,b] = sum_k A[k][j-lo-k]  * B[j-lo-k, b].
// A block computes a 128 x 128 tile of C (256 threads, 8 rows x 8 columns each) and walks the band
// in chunks of 32 steps.  Per chunk one thread issues two TMA tile loads (cp.async.bulk.tensor,
// no multicast) into a double-buffered stage: the slice of the diagonal band and the window of B
// rows the chunk touches, for all 128 batch columns (B's columns are contiguous runs of rows, so
// the window is a 2-D box of the column-major operand).  Out-of-range rows/diagonals arrive as
// zeros.  The band slice is then re-laid in shared memory ("skewed") so that the 8 coefficients a
// thread needs in one step are contiguous; in the same pass they are multiplied by factAB and
// cells whose matrix column/row falls outside the matrix are zeroed, so padding cells of the
// diagonal storage never contribute (they may hold NaN).  In the main loop a step costs two
// 128-bit loads of coefficients and a quarter of eight 128-bit loads of B for 64 multiply-adds,
// with no register shuffling: stepping index q = (row in thread) + (diagonal) for 'n', and
// q = (diagonal) - (row in thread) for 't', makes every thread row read the same B row in a step.
// Per output the terms are still added in diagonal storage order, so the EXACT mode (separate
// multiply and add) reproduces CUV's host loop (matrix_ops/spmv.cu:161-198) bit for bit, except
// that skipped cells are added as +0 (a -0 accumulator becomes +0) and a non-finite B value next
// to the band edge meets a zeroed coefficient.  A is read from HBM once per 128 batch columns and
// stays in L2 across column tiles; the kernel is bound by FP32 issue, not by memory.
#include <cuda.h>

#include "cuvdia_internal.cuh"

namespace cuvdia {

namespace pb {
constexpr int TM = 128;          // output rows per block
constexpr int TN = 128;          // batch columns per block
constexpr int KC = 32;           // steps per chunk
constexpr int NRAW = KC + 7;     // diagonals a chunk touches
constexpr int WR = 156;          // rows of the B window (>= KC + 120, = 4 * odd: conflict-free 128-bit loads)
constexpr int NCONS_WARPS = 8;      // consumer warps: the 128 x 128 tile
constexpr int NPROD_WARPS = 4;      // producer warps: TMA issue + skew pass
constexpr int THREADS = 32 * (NCONS_WARPS + NPROD_WARPS);
constexpr int RAW_FLOATS_N = TM * NRAW;     // 'n': band slice is TM rows wide
constexpr int RAW_FLOATS_T = WR * NRAW;     // 't': band slice is as wide as the B window
constexpr int BS_FLOATS = WR * TN;
constexpr int AS_FLOATS = KC * TM;
__host__ __device__ constexpr size_t align128(size_t x) { return (x + 127) / 128 * 128; }
template <bool TRANS> __host__ __device__ constexpr size_t raw_bytes() { return align128(sizeof(float) * (TRANS ? RAW_FLOATS_T : RAW_FLOATS_N)); }
__host__ __device__ constexpr size_t bs_bytes() { return align128(sizeof(float) * BS_FLOATS); }
template <bool TRANS> __host__ __device__ constexpr size_t smem_bytes() {
    return raw_bytes<TRANS>() + 2 * bs_bytes() + 2 * sizeof(float) * AS_FLOATS + 128 /*barriers*/;
}
// unroll factor of the 4-step groups in the main loop: the whole chunk for the fused arithmetic (measured 53.6 against
// 52.3 TFLOP/s with 4), half of it for the exact one (three instructions per multiply-add pair: 30.0 against 29.5)
template <bool EXACT> __host__ __device__ constexpr int group_unroll() { return EXACT ? 4 : 8; }
constexpr unsigned SPIN_LIMIT = 1u << 26;   // bounded wait on a TMA completion barrier
constexpr unsigned DRAIN_LIMIT = 1u << 22;  // second, shorter wait for copies still in flight when a warp gives up
}  // namespace pb

__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(unsigned long long* bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(unsigned long long* bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// Returns false if the barrier did not complete within the spin limit.
__device__ __forceinline__ bool mbar_wait(unsigned long long* bar, unsigned parity) {
    const unsigned addr = smem_u32(bar);
    for (unsigned it = 0; it < pb::SPIN_LIMIT; it++) {
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
__device__ __forceinline__ void mbar_drain(unsigned long long* bar, unsigned parity) {
    const unsigned addr = smem_u32(bar);
    for (unsigned it = 0; it < pb::DRAIN_LIMIT; it++) {
        unsigned done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done) : "r"(addr), "r"(parity) : "memory");
        if (done) return;
    }
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, unsigned long long* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar)) : "memory");
}

// Two multiply-adds on a packed pair of floats (the f32x2 instructions of sm_100).  FAST is one
// packed fused multiply-add.  EXACT must round the product and the sum separately: a packed
// multiply followed by two scalar adds (a packed multiply feeding a packed add is contracted into
// a fused multiply-add by the assembler even with explicit rounding modifiers, so that pairing
// cannot be used).
template <bool EXACT>
__device__ __forceinline__ void mac2(float2& acc, float2 a, float2 b) {
    if (EXACT) {
        const float2 p = __fmul2_rn(a, b);
        acc.x = __fadd_rn(acc.x, p.x);
        acc.y = __fadd_rn(acc.y, p.y);
    } else {
        acc = __ffma2_rn(a, b, acc);
    }
}

struct BandParams {
    int h, w, nd, lo;         // matrix shape, number of diagonals, first offset
    int rows_out;             // h ('n') or w ('t')
    int ncols, ldc;
    int rem;                  // lo mod 4 (non-negative): shift that keeps TMA x coordinates 16-byte aligned
    int nchunks;
    int last_groups;          // 4-step groups of the last chunk that contain steps of the band (1..KC/4)
    float fa, fc;
    int vec_c;                // C allows 128-bit accesses
    float* C;
    int* status;              // set to 1 if a TMA wait gave up
};

__device__ __forceinline__ void mbar_arrive(unsigned long long* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// Warp-uniform bounded wait: either every lane sees the phase complete or the whole warp gives up.
__device__ __forceinline__ bool warp_wait(unsigned long long* bar, unsigned parity) {
    return __all_sync(0xffffffffu, mbar_wait(bar, parity) ? 1 : 0) != 0;
}

// Roles: warps 0..7 are consumers (the 128 x 128 tile, 8 x 8 outputs per thread); warps 8..11 are
// producers (four of them: one per scheduler, so that a chunk's coefficients are ready well before the
// consumers ask for them; two were measured 4 % slower).  The producers issue the TMA loads and re-lay ("skew") each band slice into the
// coefficient buffer As while the consumers are still computing the previous chunk, so the consumers
// never meet a block-wide barrier: every hand-over is an mbarrier with a bounded wait.
//   raw        one buffer: band slice of chunk c as TMA delivers it          (raw_full / raw_free)
//   As[2]      skewed, masked, factAB-scaled coefficients of chunks c, c+1   (as_full / as_empty)
//   Bs[2]      B windows of chunks c, c+1                                    (bs_full / bs_empty)
template <bool TRANS, bool EXACT>
__global__ void __launch_bounds__(pb::THREADS, 1)
prod_band_kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB,
                 const BandParams P) {
    using namespace pb;
    // Dynamic shared memory is the only shared memory of this kernel, so it starts at the aligned
    // base of the block's window; all sub-buffers are carved by plain offsets so that the compiler
    // keeps them in the shared address space (LDS/STS, not generic loads).
    extern __shared__ __align__(1024) float smem_f[];
    constexpr int RAWF = (int)(raw_bytes<TRANS>() / sizeof(float));
    constexpr int BSF = (int)(bs_bytes() / sizeof(float));
    float* const raw = smem_f;
    float* const Bs0 = smem_f + RAWF;
    float* const As0 = smem_f + RAWF + 2 * BSF;
    unsigned long long* const bars = reinterpret_cast<unsigned long long*>(As0 + 2 * AS_FLOATS);
    unsigned long long* const raw_full = bars + 0;
    unsigned long long* const raw_free = bars + 1;
    unsigned long long* const as_full = bars + 2;     // [2]
    unsigned long long* const as_empty = bars + 4;    // [2]
    unsigned long long* const bs_full = bars + 6;     // [2]
    unsigned long long* const bs_empty = bars + 8;    // [2]

    const int tid = threadIdx.x;
    // Column tiles vary fastest across the grid: blocks that run together share one slice of the band
    // (read once from HBM) and stream different batch columns; neighbouring row tiles re-use most of
    // each other's B rows out of L2.
    const int t0 = blockIdx.y * TM;               // first output row of the tile
    const int n0 = blockIdx.x * TN;               // first batch column of the tile
    const int lane = tid & 31, warp = tid >> 5;
    const int nch = P.nchunks;

    // Chunk c covers steps q in [c*KC, (c+1)*KC).
    //  'n': q = j + k + rem           (j = row within the thread's 8, k = diagonal index)
    //       band slice rows k from c*KC - rem - 7, matrix rows from t0;
    //       B window starts at matrix row t0 + lo - rem + c*KC; a thread reads window row r0 + qq.
    //  't': q = k - j + 7 + rem
    //       band slice rows k from c*KC - rem - 7, matrix rows = the B window's rows;
    //       B window starts at matrix row t0 - lo + rem + 8 - (c+1)*KC; a thread reads window row r0 + KC-1 - qq.
    auto win_row0 = [&](int c) { return TRANS ? (t0 - P.lo + P.rem + 8 - (c + 1) * KC) : (t0 + P.lo - P.rem + c * KC); };

    if (tid == 0) {
        mbar_init(raw_full, 1);
        mbar_init(raw_free, NPROD_WARPS);
#pragma unroll
        for (int s = 0; s < 2; s++) {
            mbar_init(&as_full[s], NPROD_WARPS);
            mbar_init(&as_empty[s], NCONS_WARPS);
            mbar_init(&bs_full[s], 1);
            mbar_init(&bs_empty[s], NCONS_WARPS);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    if (warp >= NCONS_WARPS) {
        // =========================== producers ===========================
        const int pw = warp - NCONS_WARPS;                     // handles the steps qq = pw, pw + NPROD_WARPS, ...
        const bool issuer = pw == 0 && lane == 0;
        constexpr unsigned RAW_TX = sizeof(float) * (TRANS ? RAW_FLOATS_T : RAW_FLOATS_N);
        constexpr unsigned BS_TX = sizeof(float) * BS_FLOATS;
        int armed_raw = -1, armed_b0 = -1, armed_b1 = -1;      // issuer: last chunk whose copy was started, per barrier
        auto issue_raw = [&](int c) {
            mbar_expect_tx(raw_full, RAW_TX);
            tma_load_2d(raw, &mapA, TRANS ? win_row0(c) : t0, c * KC - P.rem - 7, raw_full);
            armed_raw = c;
        };
        auto issue_b = [&](int c) {
            mbar_expect_tx(&bs_full[c & 1], BS_TX);
            tma_load_2d(Bs0 + (c & 1) * BSF, &mapB, win_row0(c), n0, &bs_full[c & 1]);
            if (c & 1) armed_b1 = c; else armed_b0 = c;
        };
        // a producer that gives up: the issuing thread first waits, bounded again, for the copies it started
        auto give_up = [&]() {
            if (lane == 0 && P.status) *P.status = 1;
            if (issuer) {
                if (armed_raw >= 0) mbar_drain(raw_full, armed_raw & 1);
                if (armed_b0 >= 0) mbar_drain(&bs_full[0], (armed_b0 >> 1) & 1);
                if (armed_b1 >= 0) mbar_drain(&bs_full[1], (armed_b1 >> 1) & 1);
            }
        };
        if (issuer) {
            issue_raw(0);
            issue_b(0);
            if (nch > 1) issue_b(1);
        }
        for (int c = 0; c < nch; c++) {
            bool ok = warp_wait(raw_full, c & 1);
            if (ok && c >= 2) ok = warp_wait(&as_empty[c & 1], ((c >> 1) + 1) & 1);
            if (!ok) { give_up(); return; }
            // ---- skew: As[qq][r] = factAB * A[k][matrix row], zero where the cell is outside the matrix ----
            float* as = As0 + (c & 1) * AS_FLOATS;
            const int y0 = c * KC - P.rem - 7;
            const int xb = win_row0(c);
            const int j = lane & 7;
            // block-uniform: every cell this chunk touches lies inside the matrix
            const bool interior = TRANS ? (y0 >= 0 && y0 + NRAW <= P.nd && xb >= 0 && xb + WR <= P.h)
                                        : (y0 >= 0 && y0 + NRAW <= P.nd && xb >= 0 && xb + TM + KC <= P.w);
            constexpr int SSTEP = TRANS ? NPROD_WARPS * (WR - 1) : NPROD_WARPS * TM;
#pragma unroll
            for (int m = 0; m < TM / 32; m++) {
                const int r = lane + 32 * m;
                // slice element for (qq, r):  'n': row qq-j+7, column r;   't': row qq+j, column (r-j)+KC-1-qq
                const float* src = TRANS ? raw + (pw + j) * WR + (r - j) + KC - 1 - pw : raw + (pw - j + 7) * TM + r;
                float* dst = as + pw * TM + r;
                if (interior && P.fa == 1.f) {
#pragma unroll
                    for (int it = 0; it < KC / NPROD_WARPS; it++) dst[it * NPROD_WARPS * TM] = src[it * SSTEP];
                } else {
#pragma unroll 4
                    for (int it = 0; it < KC / NPROD_WARPS; it++) {
                        const int qq = pw + NPROD_WARPS * it;
                        bool in;
                        if (!TRANS) {
                            const int k = y0 + qq - j + 7;
                            const int jb = t0 + r + P.lo + k;               // matrix column of the cell
                            in = (unsigned)k < (unsigned)P.nd && (unsigned)jb < (unsigned)P.w;
                        } else {
                            const int k = y0 + qq + j;
                            const int i = xb + (r - j) + KC - 1 - qq;       // matrix row of the cell
                            in = (unsigned)k < (unsigned)P.nd && (unsigned)i < (unsigned)P.h;
                        }
                        float v = src[it * SSTEP];
                        if (P.fa != 1.f) v = __fmul_rn(P.fa, v);
                        dst[it * NPROD_WARPS * TM] = in ? v : 0.f;
                    }
                }
            }
            __syncwarp();
            if (lane == 0) { mbar_arrive(&as_full[c & 1]); mbar_arrive(raw_free); }
            if (issuer) {
                // the slice buffer is free once every producer warp is done with it
                if (c + 1 < nch) {
                    if (!mbar_wait(raw_free, c & 1)) { if (P.status) *P.status = 1; }
                    else issue_raw(c + 1);
                }
                // the B stage of chunk c-1 is free once the consumers are done with that chunk
                if (c >= 1 && c + 1 < nch) {
                    if (!mbar_wait(&bs_empty[(c - 1) & 1], ((c - 1) >> 1) & 1)) { if (P.status) *P.status = 1; }
                    else issue_b(c + 1);
                }
            }
            __syncwarp();
        }
        return;
    }

    // =========================== consumers ===========================
    const int rg = lane >> 4, cg = lane & 15;
    const int r0 = (warp * 2 + rg) * 8;           // this thread's 8 output rows: t0 + r0 .. t0 + r0 + 7
    // this thread's 8 columns: n0 + cg + 16*c

    // acc[jp][c] holds rows (2*jp, 2*jp+1) of column c as a packed pair
    float2 acc[4][8];
#pragma unroll
    for (int jp = 0; jp < 4; jp++)
#pragma unroll
        for (int c = 0; c < 8; c++) acc[jp][c] = make_float2(0.f, 0.f);
    if (P.fc != 0.f) {
#pragma unroll
        for (int c = 0; c < 8; c++) {
            const int col = n0 + cg + 16 * c;
#pragma unroll
            for (int j = 0; j < 8; j++) {
                const int row = t0 + r0 + j;
                if (col < P.ncols && row < P.rows_out) {
                    const float v = __fmul_rn(P.C[(size_t)col * P.ldc + row], P.fc);
                    if (j & 1) acc[j >> 1][c].y = v; else acc[j >> 1][c].x = v;
                }
            }
        }
    }

    for (int c = 0; c < nch; c++) {
        const int s = c & 1;
        bool ok = warp_wait(&as_full[s], (c >> 1) & 1);
        if (ok) ok = warp_wait(&bs_full[s], (c >> 1) & 1);
        if (!ok) { if (lane == 0 && P.status) *P.status = 1; return; }
        const float* bsp = Bs0 + s * BSF + cg * WR + (TRANS ? (r0 + KC - 4) : r0);
        const float* asp = As0 + s * AS_FLOATS + r0;
        // the steps past the band's last one (the tail of the last chunk) have zero coefficients: leave them out
        const int ng = c == nch - 1 ? P.last_groups : KC / 4;
#pragma unroll group_unroll<EXACT>()
        for (int g = 0; g < ng; g++) {
            float4 bw[8];
#pragma unroll
            for (int cc = 0; cc < 8; cc++)
                bw[cc] = *reinterpret_cast<const float4*>(bsp + cc * 16 * WR + (TRANS ? -4 * g : 4 * g));
#pragma unroll
            for (int u = 0; u < 4; u++) {
                const float4 a0 = *reinterpret_cast<const float4*>(asp + (4 * g + u) * TM);
                const float4 a1 = *reinterpret_cast<const float4*>(asp + (4 * g + u) * TM + 4);
                const float2 a[4] = {make_float2(a0.x, a0.y), make_float2(a0.z, a0.w), make_float2(a1.x, a1.y),
                                     make_float2(a1.z, a1.w)};
#pragma unroll
                for (int cc = 0; cc < 8; cc++) {
                    float b;
                    if (!TRANS) b = u == 0 ? bw[cc].x : u == 1 ? bw[cc].y : u == 2 ? bw[cc].z : bw[cc].w;
                    else        b = u == 0 ? bw[cc].w : u == 1 ? bw[cc].z : u == 2 ? bw[cc].y : bw[cc].x;
                    const float2 bb = make_float2(b, b);
#pragma unroll
                    for (int jp = 0; jp < 4; jp++) mac2<EXACT>(acc[jp][cc], a[jp], bb);
                }
            }
        }
        __syncwarp();
        if (lane == 0) { mbar_arrive(&as_empty[s]); mbar_arrive(&bs_empty[s]); }
    }

    // ---- store ----
#pragma unroll
    for (int cc = 0; cc < 8; cc++) {
        const int col = n0 + cg + 16 * cc;
        if (col >= P.ncols) continue;
        float* cp = P.C + (size_t)col * P.ldc + t0 + r0;
        if (P.vec_c && t0 + r0 + 8 <= P.rows_out) {
            *reinterpret_cast<float4*>(cp) = make_float4(acc[0][cc].x, acc[0][cc].y, acc[1][cc].x, acc[1][cc].y);
            *reinterpret_cast<float4*>(cp + 4) = make_float4(acc[2][cc].x, acc[2][cc].y, acc[3][cc].x, acc[3][cc].y);
        } else {
#pragma unroll
            for (int j = 0; j < 8; j++)
                if (t0 + r0 + j < P.rows_out) cp[j] = (j & 1) ? acc[j >> 1][cc].y : acc[j >> 1][cc].x;
        }
    }
}

// ---- host side ----------------------------------------------------------------------------------------

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode() {
    static EncodeTiledFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

bool tma_available() { return get_encode() != nullptr; }

// 2-D fp32 tensor map: dim0 (contiguous) x dim1 with a pitch in elements, box0 x box1 tile, zero fill.
int make_map_2d(CUtensorMap* m, const float* base, long long dim0, long long dim1, long long pitch, int box0, int box1) {
    EncodeTiledFn enc = get_encode();
    if (!enc) { set_last_error("cuTensorMapEncodeTiled is not available from the driver"); return CUVDIA_ERR_CUDA; }
    cuuint64_t dims[2] = {(cuuint64_t)dim0, (cuuint64_t)dim1};
    cuuint64_t strides[1] = {(cuuint64_t)pitch * sizeof(float)};
    cuuint32_t box[2] = {(cuuint32_t)box0, (cuuint32_t)box1};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(base), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { set_last_error("cuTensorMapEncodeTiled failed with code %d", (int)r); return CUVDIA_ERR_CUDA; }
    return CUVDIA_OK;
}

// The same with a TMA shared-memory swizzle of 0 (none), 32, 64 or 128 bytes (the box's inner extent in bytes must not
// exceed the swizzle span).
int make_map_2d_swizzled(CUtensorMap* m, const float* base, long long dim0, long long dim1, long long pitch, int box0,
                         int box1, int swizzle_bytes) {
    EncodeTiledFn enc = get_encode();
    if (!enc) { set_last_error("cuTensorMapEncodeTiled is not available from the driver"); return CUVDIA_ERR_CUDA; }
    cuuint64_t dims[2] = {(cuuint64_t)dim0, (cuuint64_t)dim1};
    cuuint64_t strides[1] = {(cuuint64_t)pitch * sizeof(float)};
    cuuint32_t box[2] = {(cuuint32_t)box0, (cuuint32_t)box1};
    cuuint32_t estr[2] = {1, 1};
    const CUtensorMapSwizzle sw = swizzle_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B
                                  : swizzle_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B
                                  : swizzle_bytes == 32 ? CU_TENSOR_MAP_SWIZZLE_32B : CU_TENSOR_MAP_SWIZZLE_NONE;
    CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(base), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { set_last_error("cuTensorMapEncodeTiled failed with code %d", (int)r); return CUVDIA_ERR_CUDA; }
    return CUVDIA_OK;
}

static inline bool al16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

bool prod_band_applicable(const cuvdia_plan* p, const float* A, const float* B, int ldb, int ncols) {
    // The 128 x 128 tiles walk the band 32 steps at a time: with few batch columns or a narrow band most of a
    // tile is padding, and the staged-window kernel (one pass over A, B and C) is the better fit.
    if (ncols < 64 || p->nd < 24) return false;
    return p->is_band && p->rf == 1 && al16(A) && al16(B) && p->stride % 4 == 0 && ldb % 4 == 0 &&
           get_encode() != nullptr;
}

template <bool TRANS, bool EXACT>
static int launch_band_t(const cuvdia_plan* p, const float* A, const float* B, int ldb, float* C, int ldc, int ncols,
                         float fa, float fc, cudaStream_t st) {
    using namespace pb;
    CUtensorMap mapA, mapB;
    int rc = make_map_2d(&mapA, A, p->h, p->nd, p->stride, TRANS ? WR : TM, NRAW);
    if (rc) return rc;
    rc = make_map_2d(&mapB, B, TRANS ? p->h : p->w, ncols, ldb, WR, TN);
    if (rc) return rc;
    BandParams P;
    P.h = p->h; P.w = p->w; P.nd = p->nd; P.lo = p->band_lo;
    P.rows_out = TRANS ? p->w : p->h;
    P.ncols = ncols; P.ldc = ldc;
    P.rem = ((p->band_lo % 4) + 4) % 4;
    P.nchunks = (p->nd + P.rem + 7 + KC - 1) / KC;
    P.last_groups = ((p->nd + P.rem + 7) - (P.nchunks - 1) * KC + 3) / 4;
    P.fa = fa; P.fc = fc;
    P.vec_c = (al16(C) && ldc % 4 == 0) ? 1 : 0;
    P.C = C; P.status = p->d_status;
    static bool attr_done[64] = {false};          // one flag set per template instantiation
    rc = allow_dynamic_smem(prod_band_kernel<TRANS, EXACT>, smem_bytes<TRANS>(), attr_done);
    if (rc) return rc;
    const int gx = (P.rows_out + TM - 1) / TM, gy = (ncols + TN - 1) / TN;
    if (gx > 65535) { set_last_error("too many rows for the banded kernel"); return CUVDIA_ERR_UNSUPPORTED; }
    prod_band_kernel<TRANS, EXACT><<<dim3(gy, gx), THREADS, smem_bytes<TRANS>(), st>>>(mapA, mapB, P);
    count_launch();
    return check_launch("prod_band_kernel");
}

int launch_prod_band(const cuvdia_plan* p, const float* A, const float* B, int ldb, float* C, int ldc, int ncols,
                     bool trans, float fa, float fc, int mode, cudaStream_t st) {
    const bool exact = mode == CUVDIA_MODE_EXACT;
    if (trans) return exact ? launch_band_t<true, true>(p, A, B, ldb, C, ldc, ncols, fa, fc, st)
                            : launch_band_t<true, false>(p, A, B, ldb, C, ldc, ncols, fa, fc, st);
    return exact ? launch_band_t<false, true>(p, A, B, ldb, C, ldc, ncols, fa, fc, st)
                 : launch_band_t<false, false>(p, A, B, ldb, C, ldc, ncols, fa, fc, st);
}

}  // namespace cuvdia
