// Benchmark aid (not part of libcuvdia.so): measures the FP32 issue ceiling of the current device with a
// register-resident loop, so that bench.py can put the FP32-bound DIA kernels against a measured number
// rather than a data-sheet one.  Built by __graft_entry__.build() into libbench_fp32_peak.so beside this file.
//
//   int bench_fp32_peak_tflops(int variant, float* tflops)      returns 0 or a cudaError_t
// variant 0 = a separate multiply and add per step (the EXACT arithmetic of prod), 1 = one fused multiply-add per
// step (FAST), 2 = a packed-pair multiply (f32x2 instruction of sm_100) and two scalar adds (unfused), 3 = a packed
// fused multiply-add.  TFLOP/s counts a multiply-add as 2 flops.  Blocking; allocates and frees 4 bytes.
#include <cuda_runtime.h>
#include <math.h>

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

extern "C" __attribute__((visibility("default"))) int bench_fp32_peak_tflops(int variant, float* tflops) {
    if (!tflops) return (int)cudaErrorInvalidValue;
    int dev = 0, sms = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    float* d = nullptr;
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    if (e == cudaSuccess) e = cudaMalloc(&d, sizeof(float));
    if (e == cudaSuccess) e = cudaEventCreate(&e0);
    if (e == cudaSuccess) e = cudaEventCreate(&e1);
    const int blocks = sms * 8, iters = 4096;
    float best = 0.f;
    for (int rep = 0; rep < 4 && e == cudaSuccess; rep++) {
        cudaEventRecord(e0);
        switch (variant) {
            case 0: fp32_peak_kernel<0><<<blocks, 256>>>(d, iters, 0.999f, 0.001f); break;
            case 1: fp32_peak_kernel<1><<<blocks, 256>>>(d, iters, 0.999f, 0.001f); break;
            case 2: fp32_peak_kernel<2><<<blocks, 256>>>(d, iters, 0.999f, 0.001f); break;
            default: fp32_peak_kernel<3><<<blocks, 256>>>(d, iters, 0.999f, 0.001f); break;
        }
        cudaEventRecord(e1);
        e = cudaEventSynchronize(e1);
        float ms = 0.f;
        if (e == cudaSuccess) e = cudaEventElapsedTime(&ms, e0, e1);
        const double fl = 2.0 * 16.0 * iters * 256.0 * blocks;      // 16 multiply-adds per thread and iteration
        if (rep > 0 && e == cudaSuccess) best = fmaxf(best, (float)(fl / (ms * 1e-3) / 1e12));
    }
    if (e0) cudaEventDestroy(e0);
    if (e1) cudaEventDestroy(e1);
    if (d) cudaFree(d);
    *tflops = best;
    return (int)e;
}
