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
            if (!row_ok) continue;
            for (int kk = 0; kk < kn; kk++) {
                const int off = s_off[kk];
                const float* Ak = A + (size_t)(kb + kk) * S;
                if (!TRANS) {
                    const int j = rq + off;
                    if (j < 0 || j >= w) continue;       // spmv.cu:185-189: cells outside the matrix are skipped
                    float t = Ak[r];
                    if (fa != 1.f) t = __fmul_rn(fa, t);
                    const float* Bj = B + j;
#pragma unroll
                    for (int c = 0; c < CB; c++) {
                        if (c0 + c < ncols) {
                            const float x = Bj[(size_t)(c0 + c) * ldb];
                            acc[c] = EXACT ? __fadd_rn(acc[c], __fmul_rn(t, x)) : fmaf(t, x, acc[c]);
                        }
                    }
                } else {
                    const int m = r - off;               // spmv.cu:165-177: rf consecutive rows feed one output
                    if (m < 0 || (long long)(m + 1) * rf > h) continue;
                    for (int l = 0; l < rf; l++) {
                        const int i = m * rf + l;
                        float t = Ak[i];
                        if (fa != 1.f) t = __fmul_rn(fa, t);
                        const float* Bi = B + i;
#pragma unroll
                        for (int c = 0; c < CB; c++) {
                            if (c0 + c < ncols) {
                                const float x = Bi[(size_t)(c0 + c) * ldb];
                                acc[c] = EXACT ? __fadd_rn(acc[c], __fmul_rn(t, x)) : fmaf(t, x, acc[c]);
                            }
                        }
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
    // fewer columns per thread when the grid would otherwise leave SMs idle
    const int sms = sm_count();
    int cb = 8;
    if ((long long)gx * ((ncols + 7) / 8) < 2LL * sms) cb = 4;
    if ((long long)gx * ((ncols + 3) / 4) < 2LL * sms) cb = 2;
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
