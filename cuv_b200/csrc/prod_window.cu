// prod with a DIA operand for any diagonal pattern and row factor, with the dense operand staged in
// shared memory.
//
// A block owns T consecutive output rows and CB batch columns.  Every B row those outputs can touch
// - from the smallest to the largest stored offset - is copied once into shared memory (coalesced
// along the rows of each column), laid out [column][row] so that consecutive threads read
// consecutive words (no bank conflicts); for the transposed product with a row factor the rows are
// de-interleaved by their position inside a group of row_fact rows, which keeps that property.
// Each thread then walks the diagonals in storage order for its one output row: one coefficient
// (read from global memory, coalesced along the diagonal) and CB shared-memory words per term.  A B
// value is fetched from L2 once per block instead of once per diagonal that uses it, which is what
// bounds the plain generic kernel on scattered patterns.  Per term the kernel does one shared load
// per multiply-add, so its ceiling is the shared-memory bandwidth (a quarter of the FP32 rate);
// banded row_fact-1 patterns use the register-tiled kernel in prod_band.cu instead.
// EXACT accumulates (factAB*d)*x with a separate multiply and add in storage order, bit-identical
// to CUV's host loop (matrix_ops/spmv.cu:161-198).
#include "cuvdia_internal.cuh"

namespace cuvdia {

namespace pw {
constexpr int OFFS = 256;            // offsets staged per pass
constexpr size_t SMEM_LIMIT = 200 * 1024;
}

struct WindowParams {
    int h, w, nd, S, rf;
    int ldb, ldc, ncols;
    int off_min, off_max;
    int wq;                 // positions per de-interleaved plane ('t'): window rows / rf; 'n': window rows
    int pitch;              // words per column in shared memory
    int tiles;              // row tiles of T outputs a block works through with one staged window
    int natural;            // 't' with a row factor that is a multiple of 4: rows stay in memory order (see kernel)
    float fa, fc;
    const float* A; const int* offs; const float* B; float* C;
};

template <bool TRANS, bool EXACT, int T, int CB>
__global__ void __launch_bounds__(T)
prod_window_kernel(const WindowParams P) {
    extern __shared__ __align__(16) float win[];        // [CB][pitch]
    __shared__ int s_off[pw::OFFS + 8];
    const int tid = threadIdx.x;
    const int o0 = blockIdx.x * T * P.tiles;            // first output row of the block
    const int c0 = blockIdx.y * CB;
    const int rf = P.rf;
    // first B row of the window (a multiple of rf for 't', so groups of rf rows stay together)
    // ('n' with 16-byte staging: rounded down to a multiple of 4 so that every copy is aligned)
    const int lo = TRANS ? max(0, o0 - P.off_max) * rf
                         : (P.natural ? (max(0, o0 / rf + P.off_min) & ~3) : max(0, o0 / rf + P.off_min));
    const int rows_b = TRANS ? P.h : P.w;
    const int wrows = TRANS ? P.wq * rf : P.wq;
    // ---- stage the window: element (row lo+rr, column c0+c) -> win[c*pitch + pos(rr)] ----
    // Asynchronous 4-byte copies (global -> shared without passing through registers): a thread
    // issues all of its copies back to back and waits once, so the staging is bandwidth- and not
    // latency-bound.  Rows or columns outside the operand are written as zeros (source size 0).
    // With a row factor that is a multiple of 4 the transposed product needs no de-interleaving: the rf rows of
    // a group are contiguous and 16-byte aligned, so the window keeps memory order, is staged with 16-byte copies
    // and read with 128-bit loads (consecutive threads read consecutive groups: no bank conflicts).
    // The plain product with row factor 1 reads the window in memory order anyway; with aligned operands it is staged
    // with 16-byte copies too (a quarter of the copy instructions).
    const bool natural = TRANS && P.natural;
    if (P.natural) {
        for (int c = 0; c < CB; c++) {
            const int col = c0 + c;
            const float* src = P.B + (size_t)min(col, P.ncols - 1) * P.ldb;
            const unsigned dst0 = (unsigned)__cvta_generic_to_shared(win + c * P.pitch);
            for (int q = tid; 4 * q < wrows; q += T) {
                const int row = lo + 4 * q;
                const unsigned nbytes = col < P.ncols ? 4u * (unsigned)max(0, min(4, rows_b - row)) : 0u;
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;"
                             ::"r"(dst0 + 16u * q), "l"(src + min(row, (rows_b - 1) & ~3)), "r"(nbytes) : "memory");
            }
        }
    } else
    for (int c = 0; c < CB; c++) {
        const int col = c0 + c;
        const float* src = P.B + (size_t)min(col, P.ncols - 1) * P.ldb;
        const unsigned dst0 = (unsigned)__cvta_generic_to_shared(win + c * P.pitch);
#pragma unroll 4
        for (int rr = tid; rr < wrows; rr += T) {
            const int row = lo + rr;
            const int pos = TRANS ? (rr % rf) * P.wq + rr / rf : rr;
            const unsigned nbytes = (row < rows_b && col < P.ncols) ? 4u : 0u;
            asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;"
                         ::"r"(dst0 + 4u * pos), "l"(src + min(row, rows_b - 1)), "r"(nbytes) : "memory");
        }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    const int rows_out = TRANS ? P.w : P.h;
    // When the offsets span far more rows than a tile has, the window is nearly the same for neighbouring
    // tiles: the block stages it once and works through several tiles.
    for (int rt = 0; rt < P.tiles; rt++) {
    const int o = o0 + rt * T + tid;
    const bool row_ok = o < rows_out;
    float acc[CB];
#pragma unroll
    for (int c = 0; c < CB; c++) {
        acc[c] = 0.f;
        if (P.fc != 0.f && row_ok && c0 + c < P.ncols) acc[c] = __fmul_rn(P.C[(size_t)(c0 + c) * P.ldc + o], P.fc);
    }
    const int oq = TRANS ? o : (row_ok ? o / rf : 0);
    const int oqs = row_ok ? oq : -(1 << 29);            // 'n': a row past the end makes every term fall outside the matrix
    for (int kb = 0; kb < P.nd; kb += pw::OFFS) {
        const int kn = min(pw::OFFS, P.nd - kb);
        __syncthreads();                               // window staged / previous offsets consumed
        // places past the pass's last diagonal hold an offset that no row can use
        for (int t = tid; t < kn + 8; t += T) s_off[t] = t < kn ? P.offs[kb + t] : -(1 << 29);
        __syncthreads();
        if (!TRANS) {
            // term of diagonal k: A[k][o] * B[o/rf + off_k].  The coefficients of the next eight diagonals are
            // fetched while the current eight are consumed.  A term whose cell lies outside the matrix (spmv.cu:185-189)
            // carries a negative window position and is skipped; rows past the end of the matrix and the places past
            // the last diagonal of a pass are such terms too (oqs and the padded offsets see to that), so that the
            // loop needs no other test.
            constexpr int U = 8;
            float a[U], an[U];
            int pos[U], posn[U];
            const float* Ao = P.A + (size_t)kb * P.S + o;
            auto fetch = [&](int kk, float (&av)[U], int (&pv)[U]) {
#pragma unroll
                for (int u = 0; u < U; u++) {
                    const int j = oqs + s_off[kk + u];
                    const bool ok = (unsigned)j < (unsigned)P.w;
                    pv[u] = ok ? j - lo : -1;
                    av[u] = ok ? __ldg(Ao + (size_t)(kk + u) * P.S) : 0.f;
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
                    const float* wp = win + pos[u];
                    if (CB % 2 == 0) {
                        // two columns at a time: one packed multiply (or packed fused multiply-add)
#pragma unroll
                        for (int c = 0; c < CB; c += 2) {
                            const float2 x = make_float2(wp[c * P.pitch], wp[(c + 1) * P.pitch]);
                            if (EXACT) {
                                const float2 pr = __fmul2_rn(make_float2(av, av), x);
                                acc[c] = __fadd_rn(acc[c], pr.x);
                                acc[c + 1] = __fadd_rn(acc[c + 1], pr.y);
                            } else {
                                const float2 r = __ffma2_rn(make_float2(av, av), x, make_float2(acc[c], acc[c + 1]));
                                acc[c] = r.x; acc[c + 1] = r.y;
                            }
                        }
                    } else {
#pragma unroll
                        for (int c = 0; c < CB; c++) {
                            const float x = wp[c * P.pitch];
                            acc[c] = EXACT ? __fadd_rn(acc[c], __fmul_rn(av, x)) : fmaf(av, x, acc[c]);
                        }
                    }
                }
            }
        } else {
            // term (k, l): A[k][m*rf + l] * B[m*rf + l] with m = o - off_k                  (spmv.cu:165-177)
            const int mlo = lo / rf;
            const bool vec4 = (rf % 4 == 0) && (P.S % 4 == 0) && ((reinterpret_cast<uintptr_t>(P.A) & 15) == 0);
            if (vec4) {
                // groups of four rows are fetched with one 128-bit load, one diagonal ahead
                auto fetch4 = [&](int kk, int l0, bool& valid, int& m) -> float4 {
                    m = oq - s_off[kk];
                    valid = row_ok && m >= 0 && (long long)(m + 1) * rf <= P.h;
                    if (!valid) return make_float4(0.f, 0.f, 0.f, 0.f);
                    return __ldg(reinterpret_cast<const float4*>(P.A + (size_t)(kb + kk) * P.S + (size_t)m * rf + l0));
                };
                const int nl = rf / 4;                       // 128-bit groups per diagonal
                const int total = kn * nl;
                bool vn; int mn;
                float4 an = fetch4(0, 0, vn, mn);
                for (int t = 0; t < total; t++) {
                    const int l0 = (t % nl) * 4;
                    const float4 a4 = an; const bool valid = vn; const int m = mn;
                    if (t + 1 < total) an = fetch4((t + 1) / nl, ((t + 1) % nl) * 4, vn, mn);
                    if (!valid) continue;
                    const float av[4] = {a4.x, a4.y, a4.z, a4.w};
                    if (natural) {
                        const float* wn = win + (size_t)(m - mlo) * rf + l0;
#pragma unroll
                        for (int c = 0; c < CB; c++) {
                            const float4 x4 = *reinterpret_cast<const float4*>(wn + c * P.pitch);
                            const float xv[4] = {x4.x, x4.y, x4.z, x4.w};
#pragma unroll
                            for (int u = 0; u < 4; u++) {
                                const float au = (P.fa != 1.f) ? __fmul_rn(P.fa, av[u]) : av[u];
                                acc[c] = EXACT ? __fadd_rn(acc[c], __fmul_rn(au, xv[u])) : fmaf(au, xv[u], acc[c]);
                            }
                        }
                        continue;
                    }
                    const float* wp = win + (m - mlo) + l0 * P.wq;
#pragma unroll
                    for (int u = 0; u < 4; u++) {
                        const float au = (P.fa != 1.f) ? __fmul_rn(P.fa, av[u]) : av[u];
#pragma unroll
                        for (int c = 0; c < CB; c++) {
                            const float x = wp[c * P.pitch + u * P.wq];
                            acc[c] = EXACT ? __fadd_rn(acc[c], __fmul_rn(au, x)) : fmaf(au, x, acc[c]);
                        }
                    }
                }
            } else {
                for (int kk = 0; kk < kn; kk++) {
                    const int m = oq - s_off[kk];
                    const bool valid = row_ok && m >= 0 && (long long)(m + 1) * rf <= P.h;
                    if (!valid) continue;
                    const float* Ak = P.A + (size_t)(kb + kk) * P.S + (size_t)m * rf;
                    const float* wp = win + (m - mlo);
                    for (int l = 0; l < rf; l++) {
                        float au = __ldg(Ak + l);
                        if (P.fa != 1.f) au = __fmul_rn(P.fa, au);
#pragma unroll
                        for (int c = 0; c < CB; c++) {
                            const float x = wp[c * P.pitch + l * P.wq];
                            acc[c] = EXACT ? __fadd_rn(acc[c], __fmul_rn(au, x)) : fmaf(au, x, acc[c]);
                        }
                    }
                }
            }
        }
    }
    if (row_ok) {
#pragma unroll
        for (int c = 0; c < CB; c++)
            if (c0 + c < P.ncols) P.C[(size_t)(c0 + c) * P.ldc + o] = acc[c];
    }
    }   // row tiles
}

// Window rows (per plane for 't') a block of R outputs needs.
static long long window_q(const cuvdia_plan* p, bool trans, int R) {
    const long long span = (long long)p->off_max - p->off_min;
    return trans ? (long long)R + span : ((long long)R - 1) / p->rf + 1 + span + 1;
}

// rows of the staged window for a block of R outputs: never more than the operand has (whole groups for 't')
static long long window_rows(const cuvdia_plan* p, bool trans, int R, long long* wq_out) {
    long long wq = window_q(p, trans, R);
    const long long cap = trans ? ((long long)p->h + p->rf - 1) / p->rf : p->w;
    wq = std::min(wq, cap);
    if (wq_out) *wq_out = wq;
    return trans ? wq * p->rf : wq;
}

template <bool TRANS, bool EXACT, int T, int CB>
static int launch_window_t(const cuvdia_plan* p, const float* A, const float* B, int ldb, float* C, int ldc, int ncols,
                           float fa, float fc, int tiles, cudaStream_t st) {
    WindowParams P;
    P.h = p->h; P.w = p->w; P.nd = p->nd; P.S = p->stride; P.rf = p->rf;
    P.ldb = ldb; P.ldc = ldc; P.ncols = ncols; P.off_min = p->off_min; P.off_max = p->off_max;
    long long wq = 0;
    long long wrows = window_rows(p, TRANS, T * tiles, &wq);
    P.tiles = tiles;
    const bool b_aligned = ldb % 4 == 0 && (reinterpret_cast<uintptr_t>(B) & 15) == 0;
    if (TRANS) P.natural = (p->rf % 4 == 0 && p->stride % 4 == 0 && b_aligned && (reinterpret_cast<uintptr_t>(A) & 15) == 0) ? 1 : 0;
    else       P.natural = (p->rf == 1 && b_aligned) ? 1 : 0;
    if (!TRANS && P.natural) { wq += 3; wrows += 3; }    // the window starts up to 3 rows early, on a 16-byte boundary
    P.wq = (int)wq;
    // odd pitch: columns start in different banks; the memory-order window needs 16-byte aligned columns instead
    P.pitch = P.natural ? (int)((wrows + 3) / 4 * 4) : (int)(wrows | 1);
    P.fa = fa; P.fc = fc; P.A = A; P.offs = p->d_offsets; P.B = B; P.C = C;
    const size_t smem = sizeof(float) * (size_t)P.pitch * CB;
    static bool attr_done[64] = {false};
    const int arc = allow_dynamic_smem(prod_window_kernel<TRANS, EXACT, T, CB>, pw::SMEM_LIMIT, attr_done);
    if (arc) return arc;
    const int rows_out = TRANS ? p->w : p->h;
    const int gx = (rows_out + T * tiles - 1) / (T * tiles), gy = (ncols + CB - 1) / CB;
    if (gy > 65535) { set_last_error("too many batch columns"); return CUVDIA_ERR_UNSUPPORTED; }
    prod_window_kernel<TRANS, EXACT, T, CB><<<dim3(gx, gy), T, smem, st>>>(P);
    count_launch();
    return check_launch("prod_window_kernel");
}

// Picks (T, CB, row tiles per block) by a small cost model in shared-memory wavefronts: a block pays for staging
// its window (twice the copy's wavefronts, for the latency of the fetch) and one wavefront per term, column and
// warp; the blocks of the grid are spread over the SMs.  Returns false if no window fits.
static bool window_config(const cuvdia_plan* p, bool trans, int ncols, int* T, int* CB, int* tiles) {
    const int cands[7][2] = {{1024, 4}, {512, 8}, {512, 4}, {256, 16}, {256, 8}, {128, 8}, {128, 4}};
    const long long rows_out = trans ? p->w : p->h;
    const long long terms = (long long)p->nd * (trans ? p->rf : 1);        // terms per output row
    const int sms = std::max(1, sm_count());
    double best = -1.0;
    // the transposed product reads its coefficients with a stride and wants two blocks per SM to hide that: first
    // look among the windows that leave room for two, then among all that fit
    for (int pass = 0; pass < 2 && best < 0; pass++) {
        const size_t limit = (pass == 0 && trans) ? (size_t)100 * 1024 : pw::SMEM_LIMIT;
        for (auto& c : cands) {
            if (c[1] > 8 && ncols < 64) continue;
            if (c[0] > 256 && (trans || p->rf != 1)) continue;      // the large blocks serve the plain product only
            for (int nt = 1; nt <= 8; nt *= 2) {
                if (nt > 1 && (long long)c[0] * nt > rows_out) break;
                const long long wrows = window_rows(p, trans, c[0] * nt, nullptr);
                const size_t smem = (size_t)(wrows + 8) * c[1] * sizeof(float);      // covers either pitch
                if (smem > limit) continue;
                const long long blocks = ((rows_out + (long long)c[0] * nt - 1) / ((long long)c[0] * nt)) *
                                         ((ncols + c[1] - 1) / c[1]);
                // blocks that share an SM (shared memory, 2048 threads), and the rounds the grid needs on them
                const long long bps = std::max<long long>(1, std::min<long long>((size_t)227 * 1024 / (smem + 1024), 2048 / c[0]));
                const long long rounds = (blocks + (long long)sms * bps - 1) / ((long long)sms * bps);
                // throughput: staging (twice the copy's wavefronts), one shared-memory wavefront per term, column and
                // warp, two for the coefficient load of every term and warp
                const double per_block = (double)wrows * c[1] / 16.0 + (double)nt * terms * (c[1] + 2) * (c[0] / 32);
                const double throughput = (double)((blocks + sms - 1) / sms) * per_block;
                // latency: a thread walks its terms four at a time, each group waits for its coefficients (~400 cycles; groups of eight for 'n'),
                // and a round starts with the fetch of its window (~2000 cycles)
                const double latency = (double)rounds * (2000.0 + (double)nt * (double)terms / (trans ? 4.0 : 8.0) * 400.0);
                const double cost = std::max(throughput, latency);
                if (best < 0 || cost < best * 0.999) { best = cost; *T = c[0]; *CB = c[1]; *tiles = nt; }
            }
        }
    }
    return best >= 0;
}

bool prod_window_applicable(const cuvdia_plan* p, bool trans, int ncols) {
    int T, CB, tiles;
    return window_config(p, trans, ncols, &T, &CB, &tiles);
}

int launch_prod_window(const cuvdia_plan* p, const float* A, const float* B, int ldb, float* C, int ldc, int ncols,
                       bool trans, float fa, float fc, int mode, cudaStream_t st) {
    int T = 0, CB = 0, tiles = 1;
    if (!window_config(p, trans, ncols, &T, &CB, &tiles)) { set_last_error("window does not fit"); return CUVDIA_ERR_UNSUPPORTED; }
    const bool exact = mode == CUVDIA_MODE_EXACT;
#define GO(TR, EX, TT, CC) return launch_window_t<TR, EX, TT, CC>(p, A, B, ldb, C, ldc, ncols, fa, fc, tiles, st)
#define PICK(TR, EX)                                    \
    if (T == 1024 && CB == 4) GO(TR, EX, 1024, 4);      \
    if (T == 512 && CB == 8) GO(TR, EX, 512, 8);        \
    if (T == 512 && CB == 4) GO(TR, EX, 512, 4);        \
    if (T == 256 && CB == 16) GO(TR, EX, 256, 16);      \
    if (T == 256 && CB == 8) GO(TR, EX, 256, 8);        \
    if (T == 128 && CB == 8) GO(TR, EX, 128, 8);        \
    GO(TR, EX, 128, 4)
    if (trans) { if (exact) { PICK(true, true); } else { PICK(true, false); } }
    else { if (exact) { PICK(false, true); } else { PICK(false, false); } }
#undef PICK
#undef GO
}

}  // namespace cuvdia
