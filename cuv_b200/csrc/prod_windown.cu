// prod with a DIA operand of row factor 1 and any diagonal pattern whose B window fits in shared
// memory: the staged-window kernel of prod_window.cu with its inner loop stripped to what a term needs.
//
//   'n':  C[o, b] = factC*C[o, b] + sum_k (factAB * A[k][o])         * B[o + off_k, b]   (matrix_ops/spmv.cu:179-198)
//   't':  C[o, b] = factC*C[o, b] + sum_k (factAB * A[k][o - off_k]) * B[o - off_k, b]   (spmv.cu:161-177)
//
// A block owns 512 consecutive output rows (one per thread; several such tiles when the offsets span far
// more rows than a tile) and 8 batch columns, and stages every B row those outputs can touch once
// (16-byte asynchronous copies, laid out [column][row]: consecutive threads read consecutive words).
// With one shared-memory word per multiply-add the kernel issues, per term and thread, 8 loads and
// 8 multiply-adds; everything else in the loop is overhead, and it is what bounded the general kernel
// (61 instructions per term).  Here:
//  * the pitch of a staged column is a template parameter, so a term's 8 loads share one address register
//    and differ by immediates;
//  * what a term needs beyond the thread's own row number is the same for the whole tile (offset, first
//    window row) and is read from shared memory as one broadcast word: the position is an add, the
//    "cell inside the matrix" test (spmv.cu:185-189) one unsigned compare - rows past the end of the
//    matrix and the places past a pass's last diagonal fail it by construction;
//  * the coefficients of the next eight diagonals are fetched (coalesced along the diagonal) while the
//    current eight are consumed;
//  * two columns share a packed multiply (f32x2).
// The terms of an output are added in diagonal storage order with a separate multiply and add in the
// EXACT arithmetic: bit-identical to the host loop; cells outside the matrix are skipped, never read.
#include <cuda.h>

#include "cuvdia_internal.cuh"

namespace cuvdia {

int make_map_2d(CUtensorMap* m, const float* base, long long dim0, long long dim1, long long pitch, int box0, int box1);

namespace pwn {
constexpr int T = 512;               // threads = output rows per tile
constexpr int CB = 8;                // batch columns per block
constexpr int OFFS = 256;            // diagonals per pass
constexpr int U = 8;                 // diagonals per prefetch group
}

struct WindowNParams {
    int h, w, nd, S;
    int ldb, ldc, ncols;
    int off_min, off_max;
    int wrows;              // staged rows per column (a multiple of 4, at most the pitch)
    int tiles;              // row tiles of T outputs a block works through with one staged window
    float fa, fc;
    const float* A; const int* offs; const float* B; float* C;
};

// CBK: batch columns per block (8, or 4 for windows of more than 6400 rows).
template <bool TRANS, bool EXACT, int PITCH, int CBK>
__global__ void __launch_bounds__(pwn::T)
prod_windown_kernel(const WindowNParams P) {
    using namespace pwn;
    extern __shared__ __align__(16) float win[];        // [CBK][PITCH]
    __shared__ int s_j[OFFS + U];                       // per diagonal of the pass: tile's first row + offset
    const int tid = threadIdx.x;
    const int o0 = blockIdx.x * T * P.tiles;            // first output row of the block
    const int c0 = blockIdx.y * CBK;
    const int lo = max(0, TRANS ? o0 - P.off_max : o0 + P.off_min) & ~3;      // first staged B row, on a 16-byte boundary
    const int rows_b = TRANS ? P.h : P.w, rows_out = TRANS ? P.w : P.h;
    // ---- stage the window: element (row lo+rr, column c0+c) -> win[c*PITCH + rr]; rows or columns outside the
    // operand arrive as zeros (source size 0) ----
#pragma unroll
    for (int c = 0; c < CBK; c++) {
        const int col = c0 + c;
        const float* src = P.B + (size_t)min(col, P.ncols - 1) * P.ldb;
        const unsigned dst0 = (unsigned)__cvta_generic_to_shared(win + c * PITCH);
        for (int q = tid; 4 * q < P.wrows; q += T) {
            const int row = lo + 4 * q;
            const unsigned nbytes = col < P.ncols ? 4u * (unsigned)max(0, min(4, rows_b - row)) : 0u;
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;"
                         ::"r"(dst0 + 16u * q), "l"(src + min(row, (rows_b - 1) & ~3)), "r"(nbytes) : "memory");
        }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    asm volatile("cp.async.wait_group 0;" ::: "memory");

    for (int rt = 0; rt < P.tiles; rt++) {
        const int ob = o0 + rt * T;                     // first row of the tile
        const int o = ob + tid;
        const bool row_ok = o < rows_out;
        // a row past the end of the matrix gets a row number that puts every term outside the matrix
        const int tj = row_ok ? tid : -(1 << 29);
        float acc[CBK];
#pragma unroll
        for (int c = 0; c < CBK; c++) {
            acc[c] = 0.f;
            if (P.fc != 0.f && row_ok && c0 + c < P.ncols) acc[c] = __fmul_rn(P.C[(size_t)(c0 + c) * P.ldc + o], P.fc);
        }
        for (int kb = 0; kb < P.nd; kb += OFFS) {
            const int kn = min(OFFS, P.nd - kb);
            __syncthreads();                            // window staged / previous pass consumed
            // places past the pass's last diagonal hold a value that no row can use
            for (int t = tid; t < kn + U; t += T)
                s_j[t] = t < kn ? (TRANS ? ob - P.offs[kb + t] : ob + P.offs[kb + t]) : -(1 << 29);
            __syncthreads();
            // 'n': the coefficient sits at the output's row; 't': at the B row of the term
            const float* Ao = P.A + (size_t)kb * P.S + (TRANS ? 0 : o);
            float a[U], an[U];
            int pos[U], posn[U];
            auto fetch = [&](int kk, float (&av)[U], int (&pv)[U]) {
#pragma unroll
                for (int u = 0; u < U; u++) {
                    const int j = tj + s_j[kk + u];                 // B row of the term
                    const bool ok = (unsigned)j < (unsigned)rows_b;
                    pv[u] = ok ? j - lo : -1;
                    av[u] = ok ? __ldg(Ao + (size_t)(kk + u) * P.S + (TRANS ? j : 0)) : 0.f;
                }
            };
            fetch(0, an, posn);
            for (int kk = 0; kk < kn; kk += U) {
#pragma unroll
                for (int u = 0; u < U; u++) { a[u] = an[u]; pos[u] = posn[u]; }
                if (kk + U < kn) fetch(kk + U, an, posn);
#pragma unroll
                for (int u = 0; u < U; u++) {
                    if (pos[u] < 0) continue;
                    const float av = (P.fa != 1.f) ? __fmul_rn(P.fa, a[u]) : a[u];
                    const float2 aa = make_float2(av, av);
                    const float* wp = win + pos[u];
#pragma unroll
                    for (int c = 0; c < CBK; c += 2) {
                        const float2 x = make_float2(wp[c * PITCH], wp[(c + 1) * PITCH]);
                        if (EXACT) {
                            const float2 pr = __fmul2_rn(aa, x);
                            acc[c] = __fadd_rn(acc[c], pr.x);
                            acc[c + 1] = __fadd_rn(acc[c + 1], pr.y);
                        } else {
                            const float2 r = __ffma2_rn(aa, x, make_float2(acc[c], acc[c + 1]));
                            acc[c] = r.x; acc[c + 1] = r.y;
                        }
                    }
                }
            }
        }
        if (row_ok) {
#pragma unroll
            for (int c = 0; c < CBK; c++)
                if (c0 + c < P.ncols) P.C[(size_t)(c0 + c) * P.ldc + o] = acc[c];
        }
    }
}

// ---- the plain product fed by TMA ---------------------------------------------------------------------------------
// The same block (512 output rows x 8 batch columns, one row per thread) with nothing but the terms left in the
// consumers' loop.  One more warp issues the copies (TMA, no multicast):
//  * the B window, in segments of 1024 rows x 8 columns with one mbarrier each: one bulk copy (cp.async.bulk) per
//    column and segment - a column of B is contiguous - since tile loads of 256 rows x 1 column, 152 per block,
//    took longer than the arithmetic.  The window spans every row the block's outputs can ADDRESS (first row:
//    block's first row + smallest offset, on a 16-byte boundary), whether or not it lies inside the matrix - only
//    the rows inside are copied, the others are never used - so a term's window position is the thread's row plus
//    a number that is the same for the whole block, with no clamping.  A warp waits only for the segments its next
//    eight diagonals touch: with offsets stored in ascending order the arithmetic starts when the first segment
//    has landed and runs while the rest of the window is still on its way;
//  * the coefficients, eight diagonals x 512 rows at a time, through a ring of stages (full/empty mbarriers, bounded
//    waits): a coefficient is one conflict-free shared-memory load at an immediate offset instead of an address
//    computation, a global load and a prefetch register.
// Cells outside the matrix hold padding in the diagonal storage (possibly NaN): the multiply runs on whatever is
// there, the ADD is predicated on the cell lying inside the matrix (one compare per term), so such terms leave the
// sum untouched exactly as the host loop's skip does (spmv.cu:185-189) and there is no branch in the loop.
namespace pwn {
constexpr int NDMAX = 1024;          // diagonals the per-block tables hold
constexpr int SEG = 1024;            // window rows per segment: one bulk copy per column and segment
constexpr unsigned SPIN_LIMIT = 1u << 26;
constexpr int CP = T + 8;            // transposed product: a staged diagonal holds 516 coefficients (one row of padding words)
template <bool TRANS> __host__ __device__ constexpr int coef_stage() { return TRANS ? U * CP : U * T; }
template <bool TRANS, int PITCH, int NSTA> __host__ __device__ constexpr size_t tma_smem_bytes() {
    return sizeof(float) * ((size_t)CB * PITCH + (size_t)NSTA * coef_stage<TRANS>()) +
           sizeof(int) * ((TRANS ? 2 : 1) * NDMAX + 2 * (NDMAX / U)) + 8 * ((PITCH + SEG - 1) / SEG + 2 * NSTA) + 64;
}
}  // namespace pwn

struct WindowTmaParams {
    int h, w, nd, S;
    int ldb, ldc, ncols;
    int off_min, off_max;
    const float* A;         // the diagonals' values (the transposed product copies its coefficients itself)
    int nseg;               // window segments of 1024 rows
    int wrows;              // window rows a block's threads can address (a multiple of 4, at most the pitch)
    int tiles;              // row tiles of 512 outputs a block works through with one staged window
    float fa, fc;
    const int* offs; const float* B; float* C;
    int* status;
};

__device__ __forceinline__ unsigned wn_smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ bool wn_wait(unsigned long long* bar, unsigned parity, unsigned limit) {
    const unsigned addr = wn_smem_u32(bar);
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
__device__ __forceinline__ void wn_tma_2d(void* dst, const CUtensorMap* map, int x, int y, unsigned long long* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(wn_smem_u32(dst)), "l"(map), "r"(x), "r"(y), "r"(wn_smem_u32(bar)) : "memory");
}

// TRANS: C = A^T B.  The term of output o on diagonal k is A[k][o - off_k] * B[o - off_k]: the window position is the
// thread's row MINUS the offset, and the coefficient sits at the same row of the diagonal as the B value, so a block's
// coefficients of one diagonal are 512 consecutive values starting at row (tile's first output) - off_k.  That start is
// on no particular boundary: the producer copies, per diagonal, the 516 values from the 16-byte boundary below it (one
// bulk copy, clipped to the diagonal's storage) and a thread adds the diagonal's shift (0..3 values, one more broadcast
// word per term) to its own index.
template <bool TRANS, bool EXACT, int PITCH, int NSTA, int MINB>
__global__ void __launch_bounds__(pwn::T + 32, MINB)
prod_windown_tma_kernel(const __grid_constant__ CUtensorMap mapA, const WindowTmaParams P) {
    using namespace pwn;
    constexpr int NSEG_MAX = (PITCH + SEG - 1) / SEG;
    constexpr int CSTAGE = coef_stage<TRANS>();
    extern __shared__ __align__(1024) float smem[];
    float* const win = smem;                                            // [CB][PITCH]
    float* const coef = smem + CB * PITCH;                              // 'n': [NSTA][2 halves][U][256]; 't': [NSTA][U][CP]
    int* const s_p4 = reinterpret_cast<int*>(coef + NSTA * CSTAGE);     // per diagonal: 4 * (window row of the block's first output)
    int* const s_c4 = s_p4 + NDMAX;                                     // 't': per diagonal, 4 * (its coefficients' shift, 0..3)
    int* const s_gmin = s_c4 + (TRANS ? NDMAX : 0);                     // per group of U diagonals: smallest / largest of those rows
    int* const s_gmax = s_gmin + NDMAX / U;
    unsigned long long* const wbar = reinterpret_cast<unsigned long long*>(s_gmax + NDMAX / U);   // [NSEG_MAX]
    unsigned long long* const full = wbar + NSEG_MAX;                   // [NSTA]
    unsigned long long* const empty = full + NSTA;                      // [NSTA]

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int o0 = blockIdx.x * T * P.tiles;            // first output row of the block
    const int c0 = blockIdx.y * CB;
    // first window row (may lie before the matrix), on a 16-byte boundary
    const int lo = (TRANS ? o0 - P.off_max : o0 + P.off_min) & ~3;
    const int rows_b = TRANS ? P.h : P.w, rows_out = TRANS ? P.w : P.h;
    const int ngroups = (P.nd + U - 1) / U;
    const int nstages = ngroups * P.tiles;              // coefficient stages the block consumes, tile after tile

    if (tid == 0) {
        for (int s = 0; s < P.nseg; s++) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(wn_smem_u32(&wbar[s])));
#pragma unroll
        for (int s = 0; s < NSTA; s++) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(wn_smem_u32(&full[s])));
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(wn_smem_u32(&empty[s])), "r"(T / 32));
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    // From here on the producer warp and the consumers go separate ways: the copies are under way while the consumers
    // build their tables (which need the offsets from global memory) and meet at a barrier of their own.
    if (warp != T / 32) {
        for (int k = tid; k < ngroups * U; k += T) {
            const int off = k < P.nd ? P.offs[k] : (TRANS ? P.off_max : P.off_min);
            s_p4[k] = 4 * ((TRANS ? o0 - off : o0 + off) - lo);
            if (TRANS) s_c4[k] = 4 * ((o0 - off) & 3);
        }
        asm volatile("bar.sync 1, %0;" ::"n"(T) : "memory");
        for (int g = tid; g < ngroups; g += T) {
            int mn = s_p4[g * U], mx = mn;
#pragma unroll
            for (int u = 1; u < U; u++) { mn = min(mn, s_p4[g * U + u]); mx = max(mx, s_p4[g * U + u]); }
            s_gmin[g] = mn >> 2; s_gmax[g] = mx >> 2;
        }
        asm volatile("bar.sync 1, %0;" ::"n"(T) : "memory");
    }

    if (warp == T / 32) {
        // ================= producer warp =================
        auto issue_coef = [&](int n) {                  // stage n: tile n / ngroups, diagonals U * (n % ngroups) ..
            const int s = n % NSTA;
            const int row = o0 + (n / ngroups) * T, dia = (n % ngroups) * U;
            if (!TRANS) {
                if (lane == 0) {
                    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;"
                                 ::"r"(wn_smem_u32(&full[s])), "r"((unsigned)(sizeof(float) * U * T)) : "memory");
                    wn_tma_2d(coef + s * CSTAGE, &mapA, row, dia, &full[s]);
                    wn_tma_2d(coef + s * CSTAGE + U * 256, &mapA, row + 256, dia, &full[s]);
                }
                return;
            }
            // lane u copies diagonal dia + u: the rows from the 16-byte boundary at or below (tile's first output - offset),
            // 516 of them, clipped to the diagonal's storage (rows 0 .. S-1; those past the matrix are padding nobody adds)
            int a = 0, b = 0, x4 = 0;
            if (lane < U && dia + lane < P.nd) {
                x4 = (row - P.offs[dia + lane]) & ~3;
                a = max(x4, 0); b = min(x4 + T + 4, P.S);
                if (b < a) b = a;
            }
            unsigned bytes = sizeof(float) * (unsigned)(b - a), total = bytes;
#pragma unroll
            for (int d = 16; d >= 1; d >>= 1) total += __shfl_xor_sync(0xffffffffu, total, d);
            const unsigned bar = wn_smem_u32(&full[s]);
            if (lane == 0)
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(total) : "memory");
            __syncwarp();
            if (bytes > 0)
                asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                             ::"r"(wn_smem_u32(coef + s * CSTAGE + lane * CP + (a - x4))),
                               "l"(P.A + (size_t)(dia + lane) * P.S + a), "r"(bytes), "r"(bar) : "memory");
        };
        // the first coefficient stage, then the window segment by segment, then the ring
        issue_coef(0);
        const int ncol = min(CB, P.ncols - c0);
        for (int sg = 0; sg < P.nseg; sg++) {
            // the segment's rows that lie inside the matrix: whole groups of four by bulk copy, up to three more by hand
            // (the last segment ends with the window: a column's copy must not run on into the next column's rows)
            const int r0 = lo + sg * SEG;
            const int v0 = max(r0, 0), v1 = min(min(r0 + SEG, lo + P.wrows), rows_b);
            const int n4 = v1 > v0 ? ((v1 - v0) & ~3) : 0, tail = v1 > v0 ? (v1 - v0) - n4 : 0;
            for (int t = lane; t < tail * ncol; t += 32) {
                const int c = t / tail, row = v0 + n4 + t % tail;
                win[c * PITCH + (row - lo)] = P.B[(size_t)(c0 + c) * P.ldb + row];
            }
            __syncwarp();
            const unsigned bar = wn_smem_u32(&wbar[sg]);
            if (lane == 0)
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;"
                             ::"r"(bar), "r"((unsigned)(sizeof(float) * n4 * ncol)) : "memory");
            __syncwarp();
            if (lane < ncol && n4 > 0)
                asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                             ::"r"(wn_smem_u32(win + lane * PITCH + (v0 - lo))), "l"(P.B + (size_t)(c0 + lane) * P.ldb + v0),
                               "r"((unsigned)(sizeof(float) * n4)), "r"(bar) : "memory");
            if (sg == 0)
                for (int n = 1; n < NSTA && n < nstages; n++) issue_coef(n);
        }
        for (int n = NSTA; n < nstages; n++) {
            bool ok = true;
            if (lane == 0) ok = wn_wait(&empty[n % NSTA], ((n / NSTA) - 1) & 1, SPIN_LIMIT);
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) {
                // the consumers never handed the stage back: record it, wait (bounded) for the copies under way so
                // that none lands in shared memory the block has given back, and stop
                if (lane == 0) {
                    *P.status = 8;
                    for (int n2 = n - NSTA; n2 < n; n2++) wn_wait(&full[n2 % NSTA], (n2 / NSTA) & 1, 1u << 22);
                    for (int sg = 0; sg < P.nseg; sg++) wn_wait(&wbar[sg], 0, 1u << 22);
                }
                return;
            }
            issue_coef(n);
        }
        // A segment that none of the block's (row, diagonal) pairs touches is waited for by no consumer: the warp
        // that started the copies stays until each of them has landed (bounded), so that the block cannot end - and
        // its shared memory be handed on - with a copy still on its way.
        if (lane == 0)
            for (int sg = 0; sg < P.nseg; sg++)
                if (!wn_wait(&wbar[sg], 0, SPIN_LIMIT)) { *P.status = 8; break; }
        return;
    }

    // ================= consumers =================
    const int half = tid >> 8, r = tid & 255;
    // this thread's coefficient of diagonal u: 'n' cbase[u * 256]; 't' cbase[u * CP + the diagonal's shift]
    const float* const cbase = TRANS ? coef + tid : coef + half * (U * 256) + r;
    unsigned ready = 0;                                               // window segments this warp has seen complete
    int n = 0;                                                        // coefficient stage
    for (int rt = 0; rt < P.tiles; rt++) {
        const int ob = o0 + rt * T, o = ob + tid;
        const bool row_ok = o < rows_out;
        // byte offset of window row (rt * T + tid) in column 0; a term adds the diagonal's s_p4
        const unsigned tb = 4u * (unsigned)(rt * T + tid);
        // a term is inside the matrix iff 0 <= lo + window row < w, i.e. (byte offset - offset of matrix row 0) < 4w
        const unsigned v0 = 4u * (unsigned)(-lo);
        const unsigned vlim = row_ok ? 4u * (unsigned)rows_b : 0u;
        const int wrow = rt * T + (tid & ~31);                        // the warp's first window row before the offset
        float acc[CB];
#pragma unroll
        for (int c = 0; c < CB; c++) {
            acc[c] = 0.f;
            if (P.fc != 0.f && row_ok && c0 + c < P.ncols) acc[c] = __fmul_rn(P.C[(size_t)(c0 + c) * P.ldc + o], P.fc);
        }
        for (int g = 0; g < ngroups; g++, n++) {
            // window segments the warp's rows touch in this group
            const int s_lo = (wrow + s_gmin[g]) / SEG, s_hi = (wrow + 31 + s_gmax[g]) / SEG;
            unsigned need = ((2u << s_hi) - (1u << s_lo)) & ~ready;
            while (need) {
                const int sg = __ffs(need) - 1;
                if (!wn_wait(&wbar[sg], 0, SPIN_LIMIT)) { *P.status = 8; return; }
                ready |= 1u << sg; need &= need - 1;
            }
            const int s = n % NSTA;
            if (!wn_wait(&full[s], (n / NSTA) & 1, SPIN_LIMIT)) { *P.status = 8; return; }
            const float* cs = cbase + s * CSTAGE;
            const int un = min(U, P.nd - g * U);
#pragma unroll
            for (int u = 0; u < U; u++) {
                if (u >= un) break;                                   // block-uniform: the last group may be partial
                const unsigned addr = tb + (unsigned)s_p4[g * U + u];
                const bool ok = (addr - v0) < vlim;
                float av = TRANS ? *reinterpret_cast<const float*>(reinterpret_cast<const char*>(cs + u * CP) + s_c4[g * U + u])
                                 : cs[u * 256];
                if (P.fa != 1.f) av = __fmul_rn(P.fa, av);
                const float2 aa = make_float2(av, av);
                const float* wp = reinterpret_cast<const float*>(reinterpret_cast<const char*>(win) + addr);
#pragma unroll
                for (int c = 0; c < CB; c += 2) {
                    const float2 x = make_float2(wp[c * PITCH], wp[(c + 1) * PITCH]);
                    if (EXACT) {
                        const float2 pr = __fmul2_rn(aa, x);
                        if (ok) { acc[c] = __fadd_rn(acc[c], pr.x); acc[c + 1] = __fadd_rn(acc[c + 1], pr.y); }
                    } else {
                        const float2 rr = __ffma2_rn(aa, x, make_float2(acc[c], acc[c + 1]));
                        if (ok) { acc[c] = rr.x; acc[c + 1] = rr.y; }
                    }
                }
            }
            // hand the coefficient stage back: one arrival per warp
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(wn_smem_u32(&empty[s])) : "memory");
        }
        if (row_ok) {
#pragma unroll
            for (int c = 0; c < CB; c++)
                if (c0 + c < P.ncols) P.C[(size_t)(c0 + c) * P.ldc + o] = acc[c];
        }
    }
}

// Row tiles a block works through with one staged window (1, 2, 4 or 8) and the staged rows per column; 0 if the
// kernel does not apply: row factor 1, 16-byte aligned B, at least 32 batch columns (8 per block, 4 where the window
// has more than 6400 rows), and a window of at most 12800 rows.  Several tiles per block pay when the offsets span far more rows than a tile and the grid still
// fills the GPU.
static int windown_shape(const cuvdia_plan* p, bool trans, const float* B, int ldb, int ncols, int* wrows_out) {
    using namespace pwn;
    if (p->rf != 1 || ldb % 4 != 0 || (reinterpret_cast<uintptr_t>(B) & 15) != 0 || ncols < 32) return 0;
    const long long span = (long long)p->off_max - p->off_min;
    int best = 0;
    for (int nt = 1; nt <= 8; nt *= 2) {
        const long long rows_out = trans ? p->w : p->h, rows_b = trans ? p->h : p->w;
        if (nt > 1 && (long long)T * nt > rows_out) break;
        // rows a block's outputs can touch, plus up to 3 for the 16-byte boundary the window starts on
        const long long wrows = std::min<long long>((long long)T * nt + span + 3, rows_b + 3);
        if (wrows > 12800) break;                               // 6400 rows x 8 columns, or 12800 x 4
        const long long blocks = ((rows_out + T * nt - 1) / (T * nt)) * ((ncols + CB - 1) / CB);
        if (nt > 1 && (blocks < sm_count() || span < 4LL * T * nt || wrows > 6400)) break;
        best = nt;
        *wrows_out = (int)((wrows + 3) / 4 * 4);
    }
    return best;
}

static int windown_tma_shape(const cuvdia_plan* p, bool trans, const float* A, const float* B, int ldb, int ncols,
                             int* nseg_out, int* wrows_out);

bool prod_windown_applicable(const cuvdia_plan* p, bool trans, const float* A, const float* B, int ldb, int ncols) {
    int wrows, nseg;
    if (windown_tma_shape(p, trans, A, B, ldb, ncols, &nseg, &wrows) > 0) return true;
    return windown_shape(p, trans, B, ldb, ncols, &wrows) > 0;
}

template <bool TRANS, bool EXACT, int PITCH, int CBK>
static int launch_windown_t(const WindowNParams& P, int rows_out, cudaStream_t st) {
    using namespace pwn;
    const size_t smem = sizeof(float) * ((size_t)(CBK - 1) * PITCH + (size_t)P.wrows);
    static bool attr_done[64] = {false};
    const int arc = allow_dynamic_smem(prod_windown_kernel<TRANS, EXACT, PITCH, CBK>, sizeof(float) * (size_t)CBK * PITCH, attr_done);
    if (arc) return arc;
    const int gx = (rows_out + T * P.tiles - 1) / (T * P.tiles), gy = (P.ncols + CBK - 1) / CBK;
    if (gy > 65535) { set_last_error("too many batch columns"); return CUVDIA_ERR_UNSUPPORTED; }
    prod_windown_kernel<TRANS, EXACT, PITCH, CBK><<<dim3(gx, gy), T, smem, st>>>(P);
    count_launch();
    return check_launch("prod_windown_kernel");
}

// The TMA-fed kernel serves a product when the diagonals' array and B allow TMA (16-byte aligned, pitches that
// are multiples of 4), there are at most 1024 diagonals and the rows a block can address fit its window: 5120 rows
// (one block per SM, three coefficient stages) or 2176 (two blocks per SM, two stages).  Returns the row tiles per
// block (0: does not apply) and the window segments.
static int windown_tma_shape(const cuvdia_plan* p, bool trans, const float* A, const float* B, int ldb, int ncols,
                             int* nseg_out, int* wrows_out) {
    using namespace pwn;
    auto al16 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
    // (row numbers are compared as byte offsets in 32 bits inside the kernel: matrices of up to 2^29 rows and columns)
    if (p->rf != 1 || !al16(A) || !al16(B) || ldb % 4 != 0 || p->stride % 4 != 0 || ncols < 32 || p->nd > NDMAX ||
        p->h >= (1 << 29) || p->w >= (1 << 29) || !tma_available())
        return 0;
    const long long span = (long long)p->off_max - p->off_min;
    int best = 0;
    for (int nt = 1; nt <= 8; nt *= 2) {
        const long long rows_out = trans ? p->w : p->h;
        if (nt > 1 && (long long)T * nt > rows_out) break;
        const long long wrows = (long long)T * nt + span + 3;       // every row the block's outputs can address
        if (wrows > 5120) break;
        const long long blocks = ((rows_out + T * nt - 1) / (T * nt)) * ((ncols + CB - 1) / CB);
        if (nt > 1 && (blocks < sm_count() || span < 4LL * T * nt)) break;
        best = nt;
        *nseg_out = (int)((wrows + SEG - 1) / SEG);
        *wrows_out = (int)wrows;
    }
    return best;
}

template <bool TRANS, bool EXACT, int PITCH, int NSTA, int MINB>
static int launch_windown_tma_t(const CUtensorMap& mapA, const WindowTmaParams& P, cudaStream_t st) {
    using namespace pwn;
    constexpr size_t smem = tma_smem_bytes<TRANS, PITCH, NSTA>();
    static bool attr_done[64] = {false};
    const int arc = allow_dynamic_smem(prod_windown_tma_kernel<TRANS, EXACT, PITCH, NSTA, MINB>, smem, attr_done);
    if (arc) return arc;
    const int rows_out = TRANS ? P.w : P.h;
    const int gx = (rows_out + T * P.tiles - 1) / (T * P.tiles), gy = (P.ncols + CB - 1) / CB;
    if (gy > 65535) { set_last_error("too many batch columns"); return CUVDIA_ERR_UNSUPPORTED; }
    prod_windown_tma_kernel<TRANS, EXACT, PITCH, NSTA, MINB><<<dim3(gx, gy), T + 32, smem, st>>>(mapA, P);
    count_launch();
    return check_launch("prod_windown_tma_kernel");
}

static int launch_prod_windown_tma(const cuvdia_plan* p, const float* A, const float* B, int ldb, float* C, int ldc,
                                   int ncols, bool trans, int tiles, int nseg, int wrows, float fa, float fc, int mode,
                                   cudaStream_t st) {
    using namespace pwn;
    CUtensorMap mapA;
    int rc = make_map_2d(&mapA, A, p->h, p->nd, p->stride, 256, U);
    if (rc) return rc;
    WindowTmaParams P;
    P.h = p->h; P.w = p->w; P.nd = p->nd; P.S = p->stride; P.ldb = ldb; P.ldc = ldc; P.ncols = ncols;
    P.off_min = p->off_min; P.off_max = p->off_max; P.A = A;
    P.nseg = nseg; P.wrows = (wrows + 3) & ~3; P.tiles = tiles; P.fa = fa; P.fc = fc; P.offs = p->d_offsets; P.B = B; P.C = C; P.status = p->d_status;
    const bool exact = mode == CUVDIA_MODE_EXACT;
#define GO(TR)                                                                              \
    do {                                                                                    \
        if (wrows <= 2176)                                                                  \
            return exact ? launch_windown_tma_t<TR, true, 2176, 2, 2>(mapA, P, st)          \
                         : launch_windown_tma_t<TR, false, 2176, 2, 2>(mapA, P, st);        \
        return exact ? launch_windown_tma_t<TR, true, 5120, 3, 1>(mapA, P, st)              \
                     : launch_windown_tma_t<TR, false, 5120, 3, 1>(mapA, P, st);            \
    } while (0)
    if (trans) GO(true);
    GO(false);
#undef GO
}

int launch_prod_windown(const cuvdia_plan* p, const float* A, const float* B, int ldb, float* C, int ldc, int ncols,
                        bool trans, float fa, float fc, int mode, cudaStream_t st) {
    {
        int nseg = 0, wr = 0;
        const int tiles = windown_tma_shape(p, trans, A, B, ldb, ncols, &nseg, &wr);
        if (tiles > 0) return launch_prod_windown_tma(p, A, B, ldb, C, ldc, ncols, trans, tiles, nseg, wr, fa, fc, mode, st);
    }
    WindowNParams P;
    int wrows = 0;
    P.tiles = windown_shape(p, trans, B, ldb, ncols, &wrows);
    if (P.tiles <= 0) { set_last_error("window does not fit"); return CUVDIA_ERR_UNSUPPORTED; }
    P.h = p->h; P.w = p->w; P.nd = p->nd; P.S = p->stride;
    P.ldb = ldb; P.ldc = ldc; P.ncols = ncols; P.off_min = p->off_min; P.off_max = p->off_max; P.wrows = wrows;
    P.fa = fa; P.fc = fc; P.A = A; P.offs = p->d_offsets; P.B = B; P.C = C;
    const bool exact = mode == CUVDIA_MODE_EXACT;
    // the pitch is a compile-time constant: the smallest of four that holds the window (4, 2 or 1 blocks per SM; the
    // largest with 4 instead of 8 columns per block)
#define GO(PV, CV)                                                                                      \
    do {                                                                                                \
        if (trans) return exact ? launch_windown_t<true, true, PV, CV>(P, p->w, st) : launch_windown_t<true, false, PV, CV>(P, p->w, st); \
        return exact ? launch_windown_t<false, true, PV, CV>(P, p->h, st) : launch_windown_t<false, false, PV, CV>(P, p->h, st);        \
    } while (0)
    if (wrows <= 1600) GO(1600, 8);
    if (wrows <= 3200) GO(3200, 8);
    if (wrows <= 6400) GO(6400, 8);
    GO(12800, 4);
#undef GO
}

}  // namespace cuvdia
