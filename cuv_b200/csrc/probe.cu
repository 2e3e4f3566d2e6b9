// Measures the FP32 issue ceiling of the device with a register-resident loop, so that the
// FP32-bound kernels of this library can be put against a measured number rather than a
// data-sheet one.  Used by the benchmark harness only.
#include "cuvdia_internal.cuh"

namespace cuvdia {

template <bool FUSED>
__global__ void __launch_bounds__(256)
fp32_peak_kernel(float* out, int iters, float a, float b) {
    float x[16];
#pragma unroll
    for (int i = 0; i < 16; i++) x[i] = (float)(threadIdx.x + i);
    for (int it = 0; it < iters; it++) {
#pragma unroll
        for (int i = 0; i < 16; i++) {
            if (FUSED) x[i] = fmaf(x[i], a, b);
            else x[i] = __fadd_rn(__fmul_rn(x[i], a), b);
        }
    }
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < 16; i++) s += x[i];
    if (s == 12345.678f) out[0] = s;     // never true in practice; keeps the loop alive
}

}  // namespace cuvdia

using namespace cuvdia;

extern "C" int cuvdia_fp32_peak_tflops(int fused, float* tflops) {
    CUVDIA_REQUIRE(tflops != nullptr);
    float* d = nullptr;
    cudaEvent_t e0, e1;
    CUVDIA_CUDA(cudaMalloc(&d, sizeof(float)));
    CUVDIA_CUDA(cudaEventCreate(&e0));
    CUVDIA_CUDA(cudaEventCreate(&e1));
    const int blocks = sm_count() * 8, iters = 4096;
    float best = 0.f;
    for (int rep = 0; rep < 4; rep++) {
        cudaEventRecord(e0);
        if (fused) fp32_peak_kernel<true><<<blocks, 256>>>(d, iters, 0.999f, 0.001f);
        else fp32_peak_kernel<false><<<blocks, 256>>>(d, iters, 0.999f, 0.001f);
        cudaEventRecord(e1);
        count_launch();
        CUVDIA_CUDA(cudaEventSynchronize(e1));
        float ms = 0.f;
        CUVDIA_CUDA(cudaEventElapsedTime(&ms, e0, e1));
        // one multiply-add = 2 flops, in both variants
        const double fl = 2.0 * 16.0 * iters * 256.0 * blocks;
        if (rep > 0) best = fmaxf(best, (float)(fl / (ms * 1e-3) / 1e12));
    }
    cudaEventDestroy(e0); cudaEventDestroy(e1); cudaFree(d);
    *tflops = best;
    return check_launch("fp32_peak_kernel");
}
