// prod with a DIA operand, any diagonal pattern and any row factor.
//
// One thread owns one output row and CB batch columns and walks the diagonals in storage order,
// which is the accumulation order of CUV's host code (matrix_ops/spmv.cu:161-198).  Loads of the
// diagonal values and of the dense operand are coalesced along the diagonal (consecutive threads
// read consecutive rows).  This kernel serves scattered patterns and small problems; banded
// patterns are dispatched to the tiled kernels in prod_band.cu.
#include "cuvdia_internal.cuh"

namespace cuvdia {

constexpr int PG_THREADS = 128;
constexpr int PG_OFFS = 256;   // offsets staged in shared memory per pass

// Up to four terms of one output row at once: the loads of all four (one coefficient and CB dense
// values each) are issued before the first multiply-add, so a thread keeps 4*(CB+1) loads in
// flight; the terms are still added in order u = 0..3, i.e. in storage order.
template <bool EXACT, int CB>
__device__ __forceinline__ void add_terms4(float (&acc)[CB], const float* const (&ap)[4], const float* const (&bp)[4],
                                           const bool (&ok)[4], float fa, int c0, int ncols, int ldb) {
    float t[4];
#pragma unroll
    for (int u = 0; u < 4; u++) {
        t[u] = ok[u] ? __ldg(ap[u]) : 0.f;
        if (fa != 1.f) t[u] = __fmul_rn(fa, t[u]);
    }
    float x[CB][4];
#pragma unroll
    for (int c = 0; c < CB; c++)
#pragma unroll
        for (int u = 0; u < 4; u++)
            x[c][u] = (ok[u] && c0 + c < ncols) ? __ldg(bp[u] + (size_t)(c0 + c) * ldb) : 0.f;
#pragma unroll
    for (int c = 0; c < CB; c++)
#pragma unroll
        for (int u = 0; u < 4; u++)
            if (ok[u]) acc[c] = EXACT ? __fadd_rn(acc[c], __fmul_rn(t[u], x[c][u])) : fmaf(t[u], x[c][u], acc[c]);
}

template <bool TRANS, bool EXACT, int CB>
__global__ void __launch_bounds__(PG_THREADS)
prod_generic_kernel(const float* __restrict__ A, const int* __restrict__ offs, int nd, int h, int w, int S, int rf,
                    const float* __restrict__ B, int ldb, float* __restrict__ C, int ldc, int ncols,
                    float fa, float fc) {
    __shared__ int s_off[PG_OFFS];
    const int rows_out = TRANS ? w : h;
    const int r = blockIdx.x * PG_THREADS + threadIdx.x;
    const bool row_ok = r < rows_out;
    const int rq = TRANS ? 0 : (row_ok ? r / rf : 0);
    for (int c0 = blockIdx.y * CB; c0 < ncols; c0 += gridDim.y * CB) {
        float acc[CB];
#pragma unroll
        for (int c = 0; c < CB; c++) {
            acc[c] = 0.f;
            if (fc != 0.f && row_ok && c0 + c < ncols) acc[c] = __fmul_rn(C[(size_t)(c0 + c) * ldc + r], fc);
        }
        for (int kb = 0; kb < nd; kb += PG_OFFS) {
            const int kn = min(PG_OFFS, nd - kb);
            __syncthreads();
            for (int t = threadIdx.x; t < kn; t += PG_THREADS) s_off[t] = offs[kb + t];
            __syncthreads();
            if (!TRANS || rf == 1) {
                // one term per diagonal: four diagonals per pass
                for (int kk = 0; kk < kn; kk += 4) {
                    const float* ap[4];
                    const float* bp[4];
                    bool ok[4];
#pragma unroll
                    for (int u = 0; u < 4; u++) {
                        const int k = kk + u;
                        const int off = k < kn ? s_off[k] : 0;
                        // 'n': matrix cell (r, r/rf + off);  't' with rf 1: cell (r - off, r)   (spmv.cu:165-198)
                        const int x = TRANS ? r - off : rq + off;
                        ok[u] = row_ok && k < kn && x >= 0 && x < (TRANS ? h : w);
                        const int i = TRANS ? x : r;                    // row of the cell = index into the diagonal
                        ap[u] = A + (size_t)(kb + k) * S + (ok[u] ? i : 0);
                        bp[u] = B + (ok[u] ? x : 0);
                    }
                    add_terms4<EXACT, CB>(acc, ap, bp, ok, fa, c0, ncols, ldb);
                }
            } else {
                // transposed with a row factor: rf consecutive rows of a diagonal feed one output
                for (int kk = 0; kk < kn; kk++) {
                    const int m = r - s_off[kk];
                    const bool valid = row_ok && m >= 0 && (long long)(m + 1) * rf <= h;
                    const size_t i0 = valid ? (size_t)m * rf : 0;
                    for (int l0 = 0; l0 < rf; l0 += 4) {
                        const float* ap[4];
                        const float* bp[4];
                        bool ok[4];
#pragma unroll
                        for (int u = 0; u < 4; u++) {
                            ok[u] = valid && l0 + u < rf;
                            ap[u] = A + (size_t)(kb + kk) * S + (ok[u] ? i0 + l0 + u : 0);
                            bp[u] = B + (ok[u] ? i0 + l0 + u : 0);
                        }
                        add_terms4<EXACT, CB>(acc, ap, bp, ok, fa, c0, ncols, ldb);
                    }
                }
            }
        }
        if (row_ok) {
#pragma unroll
            for (int c = 0; c < CB; c++)
                if (c0 + c < ncols) C[(size_t)(c0 + c) * ldc + r] = acc[c];
        }
    }
}

template <bool TRANS, bool EXACT>
static int launch_generic_t(const cuvdia_plan* p, const float* A, const float* B, int ldb, float* C, int ldc,
                            int ncols, float fa, float fc, cudaStream_t st) {
    const int rows_out = TRANS ? p->w : p->h;
    const int gx = (rows_out + PG_THREADS - 1) / PG_THREADS;
    // fewer columns per thread when the grid would otherwise leave the SMs short of warps to hide
    // the latency of the scattered loads (aim for about 8 blocks of 128 threads per SM)
    const int sms = sm_count();
    int cb = 8;
    if ((long long)gx * ((ncols + 7) / 8) < 8LL * sms) cb = 4;
    if ((long long)gx * ((ncols + 3) / 4) < 8LL * sms) cb = 2;
    if (ncols == 1) cb = 1;
    const int gy = std::min(65535, (ncols + cb - 1) / cb);
    dim3 grid(gx, gy), block(PG_THREADS);
#define LAUNCH(CBV)                                                                                          \
    prod_generic_kernel<TRANS, EXACT, CBV><<<grid, block, 0, st>>>(A, p->d_offsets, p->nd, p->h, p->w,       \
                                                                   p->stride, p->rf, B, ldb, C, ldc, ncols, fa, fc)
    switch (cb) {
        case 8: LAUNCH(8); break;
        case 4: LAUNCH(4); break;
        case 2: LAUNCH(2); break;
        default: LAUNCH(1); break;
    }
#undef LAUNCH
    count_launch();
    return check_launch("prod_generic_kernel");
}

int launch_prod_generic(const cuvdia_plan* p, const float* A, const float* B, int ldb, float* C, int ldc, int ncols,
                        bool trans, float fa, float fc, int mode, cudaStream_t st) {
    const bool exact = mode == CUVDIA_MODE_EXACT;
    if (trans) return exact ? launch_generic_t<true, true>(p, A, B, ldb, C, ldc, ncols, fa, fc, st)
                            : launch_generic_t<true, false>(p, A, B, ldb, C, ldc, ncols, fa, fc, st);
    return exact ? launch_generic_t<false, true>(p, A, B, ldb, C, ldc, ncols, fa, fc, st)
                 : launch_generic_t<false, false>(p, A, B, ldb, C, ldc, ncols, fa, fc, st);
}

}  // namespace cuvdia
