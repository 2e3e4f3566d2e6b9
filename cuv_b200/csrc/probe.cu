// Measures the FP32 issue ceiling of the device with a register-resident loop, so that the
// FP32-bound kernels of this library can be put against a measured number rather than a
// data-sheet one.  Used by the benchmark harness only.
#include "cuvdia_internal.cuh"

namespace cuvdia {

// One warp polls an mbarrier that is initialised for one arrival and never gets it, the way the TMA kernels
// poll theirs, and gives up after max_polls polls with a code in the health word.
__global__ void selftest_wait_kernel(int* status, unsigned max_polls) {
    __shared__ unsigned long long bar;
    const unsigned b = (unsigned)__cvta_generic_to_shared(&bar);
    if (threadIdx.x == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(b));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();
    bool done = false;
    for (unsigned it = 0; it < max_polls && !done; it++) {
        unsigned d;
        asm volatile(
            "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(d) : "r"(b), "r"(0u) : "memory");
        done = d != 0;
    }
    if (!done && threadIdx.x == 0 && status) *status = 9;
}

int launch_selftest_wait(int* status, unsigned max_polls, cudaStream_t st) {
    selftest_wait_kernel<<<1, 32, 0, st>>>(status, max_polls);
    count_launch();
    return check_launch("selftest_wait_kernel");
}

// VARIANT 0: mul + add, 1: fused multiply-add, 2: packed-pair multiply (f32x2) + two scalar adds,
// 3: fused multiply-add on packed pairs
template <int VARIANT>
__global__ void __launch_bounds__(256)
fp32_peak_kernel(float* out, int iters, float a, float b) {
    float2 x[8];
#pragma unroll
    for (int i = 0; i < 8; i++) x[i] = make_float2((float)(threadIdx.x + i), (float)(threadIdx.x - i));
    const float2 a2 = make_float2(a, a), b2 = make_float2(b, b);
    for (int it = 0; it < iters; it++) {
#pragma unroll
        for (int i = 0; i < 8; i++) {
            if (VARIANT == 0) { x[i].x = __fadd_rn(__fmul_rn(x[i].x, a), b); x[i].y = __fadd_rn(__fmul_rn(x[i].y, a), b); }
            else if (VARIANT == 1) { x[i].x = fmaf(x[i].x, a, b); x[i].y = fmaf(x[i].y, a, b); }
            else if (VARIANT == 2) { const float2 p = __fmul2_rn(x[i], a2); x[i].x = __fadd_rn(p.x, b); x[i].y = __fadd_rn(p.y, b); }
            else x[i] = __ffma2_rn(x[i], a2, b2);
        }
    }
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < 8; i++) s += x[i].x + x[i].y;
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
        switch (fused) {
            case 0: fp32_peak_kernel<0><<<blocks, 256>>>(d, iters, 0.999f, 0.001f); break;
            case 1: fp32_peak_kernel<1><<<blocks, 256>>>(d, iters, 0.999f, 0.001f); break;
            case 2: fp32_peak_kernel<2><<<blocks, 256>>>(d, iters, 0.999f, 0.001f); break;
            default: fp32_peak_kernel<3><<<blocks, 256>>>(d, iters, 0.999f, 0.001f); break;
        }
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
