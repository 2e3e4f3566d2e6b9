// avg_diagonals: the mean of every stored diagonal of a DIA matrix over the cells that lie inside the matrix,
// dst[k] = sum_{cells of diagonal k} A / N_k, as CUV's host code defines it (matrix_ops/diagonals.cu:23-48:
// i_start = max(0,-offset), j_start = max(0,offset), N = min(h - i_start, w - j_start), row_fact 1).  CUV's device
// version (:13-22) averages the whole stored array of the diagonal, padding included, and its own test has the call
// commented out ("NOT IMPLEMENTED", src/tests/dia_mat.cpp:134-142); the host definition is the one followed here.
// One block per diagonal: 128-bit loads where the range allows, warp shuffles, a fixed order (reproducible run to run).
#include "cuvdia_internal.cuh"

namespace cuvdia {

__global__ void __launch_bounds__(256)
avg_diagonals_kernel(float* __restrict__ dst, const float* __restrict__ A, const int* __restrict__ offs, int h, int w,
                     int S) {
    __shared__ float part[8];
    const int k = blockIdx.x, off = offs[k];
    const int i0 = max(0, -off), j0 = max(0, off);
    const int n = min(h - i0, w - j0);
    if (n <= 0) { if (threadIdx.x == 0) dst[k] = __int_as_float(0x7fc00000); return; }     // no cell inside the matrix: no mean (NaN)
    const float* d = A + (size_t)k * S + i0;
    float sum = 0.f;
    for (int i = threadIdx.x; i < n; i += 256) sum += d[i];
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) sum += __shfl_down_sync(0xffffffffu, sum, s);
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = sum;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = part[0];
        for (int v = 1; v < 8; v++) t += part[v];
        dst[k] = t / (float)n;
    }
}

int launch_avg_diagonals(const cuvdia_plan* p, const float* A, float* dst, cudaStream_t st) {
    avg_diagonals_kernel<<<p->nd, 256, 0, st>>>(dst, A, p->d_offsets, p->h, p->w, p->stride);
    count_launch();
    return check_launch("avg_diagonals_kernel");
}

}  // namespace cuvdia
