// densedense_to_dia for any diagonal pattern and row factor.
//
// C_dia[k][i] = factC*C_dia[k][i] + factAB * sum_b A[i,b] * B[i/rf + off_k, b]
//
// A block owns 128 consecutive rows and KD diagonals; each thread keeps KD running sums in
// registers while it streams over (its share of) the batch, so every A value is loaded once per KD
// products.  Loads are coalesced along the diagonal.  When rows x diagonals give too few blocks
// to fill the GPU the batch is split over blockIdx.z; the partial sums go to plan-owned scratch
// and a second kernel adds them in split order, so the result does not depend on scheduling.
// Only cells inside a diagonal's valid range are ever read or written
// (matrix_ops/densedense_to_sparse.cu:104-119).
#include "cuvdia_internal.cuh"

namespace cuvdia {

constexpr int DG_THREADS = 128;

__device__ __forceinline__ void dd_store(float* c, float s, float fa, float fc) {
    if (fa != 1.f) s = __fmul_rn(fa, s);
    *c = (fc != 0.f) ? __fadd_rn(__fmul_rn(fc, *c), s) : s;
}

template <int KD>
__global__ void __launch_bounds__(DG_THREADS)
dd2dia_generic_kernel(float* __restrict__ Cv, const int* __restrict__ offs, int nd, int h, int w, int S, int rf,
                      const float* __restrict__ A, int lda, const float* __restrict__ B, int ldb, int ncols,
                      float fa, float fc, int nsplit, float* __restrict__ partial) {
    const int i = blockIdx.x * DG_THREADS + threadIdx.x;
    const int k0 = blockIdx.y * KD;
    const int z = blockIdx.z;
    const int b0 = (int)((long long)ncols * z / nsplit), b1 = (int)((long long)ncols * (z + 1) / nsplit);
    if (i >= h) return;
    const int iq = i / rf;
    int j[KD];
    bool ok[KD];
    float acc[KD];
#pragma unroll
    for (int kk = 0; kk < KD; kk++) {
        const int k = k0 + kk;
        j[kk] = 0; ok[kk] = false; acc[kk] = 0.f;
        if (k < nd) {
            const int jj = iq + offs[k];
            ok[kk] = jj >= 0 && jj < w;
            j[kk] = ok[kk] ? jj : 0;
        }
    }
    const float* Ap = A + i;
    int b = b0;
    for (; b + 4 <= b1; b += 4) {
        float x[4];
#pragma unroll
        for (int u = 0; u < 4; u++) x[u] = Ap[(size_t)(b + u) * lda];
#pragma unroll
        for (int kk = 0; kk < KD; kk++) {
            if (ok[kk]) {
                const float* Bp = B + j[kk];
                float y[4];
#pragma unroll
                for (int u = 0; u < 4; u++) y[u] = Bp[(size_t)(b + u) * ldb];
#pragma unroll
                for (int u = 0; u < 4; u++) acc[kk] = fmaf(x[u], y[u], acc[kk]);
            }
        }
    }
    for (; b < b1; b++) {
        const float x = Ap[(size_t)b * lda];
#pragma unroll
        for (int kk = 0; kk < KD; kk++)
            if (ok[kk]) acc[kk] = fmaf(x, B[j[kk] + (size_t)b * ldb], acc[kk]);
    }
#pragma unroll
    for (int kk = 0; kk < KD; kk++) {
        if (!ok[kk]) continue;
        const size_t cell = (size_t)(k0 + kk) * S + i;
        if (nsplit == 1) dd_store(Cv + cell, acc[kk], fa, fc);
        else partial[(size_t)z * nd * S + cell] = acc[kk];
    }
}

// Adds the nsplit partial sums of every valid cell in split order and applies the factors.
__global__ void dd2dia_combine_kernel(float* __restrict__ Cv, const int* __restrict__ offs, int nd, int h, int w,
                                      int S, int rf, float fa, float fc, int nsplit,
                                      const float* __restrict__ partial) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= h) return;
    for (int k = blockIdx.y; k < nd; k += gridDim.y) {
        const int jj = i / rf + offs[k];
        if (jj < 0 || jj >= w) continue;
        const size_t cell = (size_t)k * S + i;
        float s = 0.f;
        for (int z = 0; z < nsplit; z++) s += partial[(size_t)z * nd * S + cell];
        dd_store(Cv + cell, s, fa, fc);
    }
}

int ensure_plan_scratch(cuvdia_plan* p, size_t floats, cudaStream_t st) {
    if (p->scratch_floats >= floats) return CUVDIA_OK;
    if (p->scratch) {
        CUVDIA_CUDA(cudaStreamSynchronize(st));
        CUVDIA_CUDA(cudaFree(p->scratch));
        p->scratch = nullptr; p->scratch_floats = 0;
    }
    CUVDIA_CUDA(cudaMalloc(&p->scratch, floats * sizeof(float)));
    p->scratch_floats = floats;
    return CUVDIA_OK;
}

int launch_dd2dia_combine(const cuvdia_plan* p, float* Cv, float fa, float fc, int nsplit, const float* partial,
                          cudaStream_t st) {
    dim3 g2((p->h + 255) / 256, std::min(p->nd, 65535));
    dd2dia_combine_kernel<<<g2, 256, 0, st>>>(Cv, p->d_offsets, p->nd, p->h, p->w, p->stride, p->rf, fa, fc, nsplit,
                                              partial);
    count_launch();
    return check_launch("dd2dia_combine_kernel");
}

int launch_dd2dia_generic(cuvdia_plan* p, float* Cv, const float* A, int lda, const float* B, int ldb, int ncols,
                          float fa, float fc, cudaStream_t st) {
    constexpr int KD = 8;
    const int gx = (p->h + DG_THREADS - 1) / DG_THREADS;
    const int gy = (p->nd + KD - 1) / KD;
    if (gy > 65535) { set_last_error("num_dia too large for densedense_to_dia"); return CUVDIA_ERR_UNSUPPORTED; }
    int nsplit = 1;
    const long long ctas = (long long)gx * gy, want = 4LL * sm_count();
    if (ctas < want) nsplit = (int)std::min<long long>((want + ctas - 1) / ctas, std::max(1, ncols / 64));
    nsplit = std::max(1, std::min(nsplit, 64));
    float* partial = nullptr;
    if (nsplit > 1) {
        int rc = ensure_plan_scratch(p, (size_t)nsplit * p->nd * p->stride, st);
        if (rc) return rc;
        partial = p->scratch;
    }
    dim3 grid(gx, gy, nsplit);
    dd2dia_generic_kernel<KD><<<grid, DG_THREADS, 0, st>>>(Cv, p->d_offsets, p->nd, p->h, p->w, p->stride, p->rf, A,
                                                           lda, B, ldb, ncols, fa, fc, nsplit, partial);
    count_launch();
    int rc = check_launch("dd2dia_generic_kernel");
    if (rc) return rc;
    if (nsplit > 1) rc = launch_dd2dia_combine(p, Cv, fa, fc, nsplit, partial, st);
    return rc;
}

}  // namespace cuvdia
