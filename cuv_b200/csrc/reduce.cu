// reduce_to_col / reduce_to_row: dst = factOld*dst + factNew*functor(src) along one axis.
//
// src is n_strided lines of n_contig contiguous floats.  After CUV's layout normalisation
// (matrix_ops/matrix_ops_reduce.cu:348-379) there are two memory patterns:
//   across lines  (over_strided): one output per contiguous position; threads own 4 adjacent
//                 outputs and read 128-bit vectors, blocks split the lines among them;
//   along lines   (!over_strided): one output per line; a warp (short lines) or a block (long
//                 lines, optionally several blocks per line) reads the line with 128-bit loads and
//                 folds it with warp shuffles.
// When several blocks share an output their partial results go to a per-stream workspace and a
// second kernel folds them in a fixed order, so results are reproducible run to run.
// Functor semantics follow tensor_ops/functors.hpp (rv/rr steps :453-516, initial values :599-644)
// and the post-processing of reduce_switch (matrix_ops_reduce.cu:304-338).
#include <cfloat>

#include "cuvdia_internal.cuh"

namespace cuvdia {

template <int RF> struct Fn {
    static constexpr bool is_arg = (RF == CUVDIA_RF_ARGMAX || RF == CUVDIA_RF_ARGMIN);
    __device__ static float init() {
        if (RF == CUVDIA_RF_MAX || RF == CUVDIA_RF_ARGMAX) return -FLT_MAX;
        if (RF == CUVDIA_RF_MIN || RF == CUVDIA_RF_ARGMIN) return FLT_MAX;
        if (RF == CUVDIA_RF_LOGADDEXP || RF == CUVDIA_RF_ADDEXP) return -INFINITY;
        return 0.f;
    }
    __device__ static float lae(float t, float u) {          // functors.hpp:520-531
        const float d = t - u;
        if (d > 0) return t + log1pf(expf(-d));
        else if (d <= 0) return u + log1pf(expf(d));
        return t + u;
    }
    // fold a raw value
    __device__ static void rv(float& r, int& idx, float v, int j) {
        if (RF == CUVDIA_RF_ADD || RF == CUVDIA_RF_MEAN) r = r + v;
        else if (RF == CUVDIA_RF_ADD_SQUARED) r = r + v * v;
        else if (RF == CUVDIA_RF_MAX) r = r > v ? r : v;
        else if (RF == CUVDIA_RF_MIN) r = r < v ? r : v;
        else if (RF == CUVDIA_RF_ARGMAX) { if (v > r) { r = v; idx = j; } }
        else if (RF == CUVDIA_RF_ARGMIN) { if (v < r) { r = v; idx = j; } }
        else if (RF == CUVDIA_RF_MULT) r = r + logf(v);
        else r = lae(r, v);
    }
    // fold a partial result; for the index functors ties go to the smaller index, which is what a
    // sequential scan in index order returns
    __device__ static void rr(float& r, int& idx, float r2, int idx2) {
        if (RF == CUVDIA_RF_ADD || RF == CUVDIA_RF_MEAN || RF == CUVDIA_RF_ADD_SQUARED || RF == CUVDIA_RF_MULT)
            r = r + r2;
        else if (RF == CUVDIA_RF_MAX) r = r > r2 ? r : r2;
        else if (RF == CUVDIA_RF_MIN) r = r < r2 ? r : r2;
        else if (RF == CUVDIA_RF_ARGMAX) { if (r2 > r || (r2 == r && idx2 < idx)) { r = r2; idx = idx2; } }
        else if (RF == CUVDIA_RF_ARGMIN) { if (r2 < r || (r2 == r && idx2 < idx)) { r = r2; idx = idx2; } }
        else r = lae(r, r2);
    }
    __device__ static void finish(float* dst, float val, int idx, float fnew, float fold, float n_red) {
        if (is_arg) { *dst = (float)idx; return; }
        float r = (fold != 0.f) ? fold * *dst + fnew * val : fnew * val;
        if (RF == CUVDIA_RF_MEAN) r = r / n_red;
        if (RF == CUVDIA_RF_MULT || RF == CUVDIA_RF_ADDEXP) r = expf(r);
        *dst = r;
    }
};

// ------------------------------------------------------------------------------------------------
// across lines: outputs along the contiguous axis
// ------------------------------------------------------------------------------------------------
constexpr int RA_THREADS = 128;

template <int RF, int VEC>
__global__ void __launch_bounds__(RA_THREADS)
reduce_across_kernel(float* __restrict__ dst, const float* __restrict__ src, long long n_contig, int n_strided,
                     float fnew, float fold, int nsplit, float* __restrict__ pval, int* __restrict__ pidx) {
    using F = Fn<RF>;
    const long long o = ((long long)blockIdx.x * RA_THREADS + threadIdx.x) * VEC;
    if (o >= n_contig) return;
    const int z = blockIdx.y;
    const int j0 = (int)((long long)n_strided * z / nsplit), j1 = (int)((long long)n_strided * (z + 1) / nsplit);
    float val[VEC];
    int idx[VEC];
#pragma unroll
    for (int v = 0; v < VEC; v++) { val[v] = F::init(); idx[v] = 0; }
    const float* p = src + o;
    int j = j0;
    if (VEC == 4) {
        for (; j + 4 <= j1; j += 4) {
            float4 x[4];
#pragma unroll
            for (int u = 0; u < 4; u++) x[u] = __ldg(reinterpret_cast<const float4*>(p + (size_t)(j + u) * n_contig));
#pragma unroll
            for (int u = 0; u < 4; u++) {
                F::rv(val[0], idx[0], x[u].x, j + u); F::rv(val[1], idx[1], x[u].y, j + u);
                F::rv(val[2], idx[2], x[u].z, j + u); F::rv(val[3], idx[3], x[u].w, j + u);
            }
        }
        for (; j < j1; j++) {
            const float4 x = __ldg(reinterpret_cast<const float4*>(p + (size_t)j * n_contig));
            F::rv(val[0], idx[0], x.x, j); F::rv(val[1], idx[1], x.y, j);
            F::rv(val[2], idx[2], x.z, j); F::rv(val[3], idx[3], x.w, j);
        }
    } else {
        for (; j + 4 <= j1; j += 4) {
            float x[4];
#pragma unroll
            for (int u = 0; u < 4; u++) x[u] = __ldg(p + (size_t)(j + u) * n_contig);
#pragma unroll
            for (int u = 0; u < 4; u++) F::rv(val[0], idx[0], x[u], j + u);
        }
        for (; j < j1; j++) F::rv(val[0], idx[0], __ldg(p + (size_t)j * n_contig), j);
    }
#pragma unroll
    for (int v = 0; v < VEC; v++) {
        if (nsplit == 1) F::finish(dst + o + v, val[v], idx[v], fnew, fold, (float)n_strided);
        else {
            pval[(size_t)z * n_contig + o + v] = val[v];
            if (F::is_arg) pidx[(size_t)z * n_contig + o + v] = idx[v];
        }
    }
}

// second stage for both patterns: fold nsplit partials per output in split order
template <int RF>
__global__ void reduce_combine_kernel(float* __restrict__ dst, long long n_out, float fnew, float fold, int nsplit,
                                      const float* __restrict__ pval, const int* __restrict__ pidx, float n_red) {
    using F = Fn<RF>;
    const long long o = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (o >= n_out) return;
    float val = pval[o];
    int idx = F::is_arg ? pidx[o] : 0;
    for (int z = 1; z < nsplit; z++)
        F::rr(val, idx, pval[(size_t)z * n_out + o], F::is_arg ? pidx[(size_t)z * n_out + o] : 0);
    F::finish(dst + o, val, idx, fnew, fold, n_red);
}

// ------------------------------------------------------------------------------------------------
// along lines: one output per line
// ------------------------------------------------------------------------------------------------
template <int RF>
__device__ __forceinline__ void warp_fold(float& val, int& idx) {
    using F = Fn<RF>;
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) {
        const float v2 = __shfl_down_sync(0xffffffffu, val, d);
        const int i2 = __shfl_down_sync(0xffffffffu, idx, d);
        F::rr(val, idx, v2, i2);
    }
}

// thread-level scan of [lo, hi) of one line with stride `step` threads; VEC==4 needs 16-byte aligned lines
template <int RF, int VEC>
__device__ __forceinline__ void line_scan(const float* __restrict__ line, long long lo, long long hi, int tid, int step,
                                          float& val, int& idx) {
    using F = Fn<RF>;
    if (VEC == 4) {
#pragma unroll 4
        for (long long j = lo + (long long)tid * 4; j < hi; j += (long long)step * 4) {
            if (j + 4 <= hi) {
                const float4 x = __ldg(reinterpret_cast<const float4*>(line + j));
                F::rv(val, idx, x.x, (int)j); F::rv(val, idx, x.y, (int)j + 1);
                F::rv(val, idx, x.z, (int)j + 2); F::rv(val, idx, x.w, (int)j + 3);
            } else {
                for (long long t = j; t < hi; t++) F::rv(val, idx, __ldg(line + t), (int)t);
            }
        }
    } else {
        for (long long j = lo + tid; j < hi; j += step) F::rv(val, idx, __ldg(line + j), (int)j);
    }
}

// a warp per line
template <int RF, int VEC>
__global__ void __launch_bounds__(256)
reduce_along_warp_kernel(float* __restrict__ dst, const float* __restrict__ src, long long n_contig, int n_strided,
                         float fnew, float fold) {
    using F = Fn<RF>;
    const int lane = threadIdx.x & 31;
    const long long line = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (line >= n_strided) return;
    float val = F::init();
    int idx = 0;
    line_scan<RF, VEC>(src + line * n_contig, 0, n_contig, lane, 32, val, idx);
    warp_fold<RF>(val, idx);
    if (lane == 0) F::finish(dst + line, val, idx, fnew, fold, (float)n_contig);
}

// a block (or nsplit blocks) per line
template <int RF, int VEC>
__global__ void __launch_bounds__(256)
reduce_along_block_kernel(float* __restrict__ dst, const float* __restrict__ src, long long n_contig, int n_strided,
                          float fnew, float fold, int nsplit, float* __restrict__ pval, int* __restrict__ pidx) {
    using F = Fn<RF>;
    __shared__ float s_val[8];
    __shared__ int s_idx[8];
    const int line = blockIdx.y, z = blockIdx.x;
    // split points are multiples of 4 so vector loads stay aligned
    const long long q = (n_contig + 3) / 4;
    const long long lo = (q * z / nsplit) * 4, hi = min(n_contig, (q * (z + 1) / nsplit) * 4);
    float val = F::init();
    int idx = 0;
    line_scan<RF, VEC>(src + (long long)line * n_contig, lo, hi, threadIdx.x, 256, val, idx);
    warp_fold<RF>(val, idx);
    if ((threadIdx.x & 31) == 0) { s_val[threadIdx.x >> 5] = val; s_idx[threadIdx.x >> 5] = idx; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int wv = 1; wv < 8; wv++) F::rr(val, idx, s_val[wv], s_idx[wv]);
        if (nsplit == 1) F::finish(dst + line, val, idx, fnew, fold, (float)n_contig);
        else {
            pval[(size_t)z * n_strided + line] = val;
            if (F::is_arg) pidx[(size_t)z * n_strided + line] = idx;
        }
    }
}

// ---- short lines ------------------------------------------------------------------------------------
// along lines shorter than a warp's reach: LPL lanes per line, 32/LPL lines per warp, so a warp
// still reads one contiguous run of memory with all lanes busy
template <int RF, int VEC, int LPL>
__global__ void __launch_bounds__(256)
reduce_along_subwarp_kernel(float* __restrict__ dst, const float* __restrict__ src, long long n_contig, int n_strided,
                            float fnew, float fold) {
    using F = Fn<RF>;
    const int lane = threadIdx.x & 31, sub = lane % LPL;
    const long long warp = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const long long line = warp * (32 / LPL) + lane / LPL;
    float val = F::init();
    int idx = 0;
    if (line < n_strided) line_scan<RF, VEC>(src + line * n_contig, 0, n_contig, sub, LPL, val, idx);
#pragma unroll
    for (int d = LPL / 2; d > 0; d >>= 1) {
        const float v2 = __shfl_down_sync(0xffffffffu, val, d, LPL);
        const int i2 = __shfl_down_sync(0xffffffffu, idx, d, LPL);
        F::rr(val, idx, v2, i2);
    }
    if (sub == 0 && line < n_strided) F::finish(dst + line, val, idx, fnew, fold, (float)n_contig);
}

// across lines when a line is at most 256 floats (NV = n_contig/4 vectors, a power of two): thread t
// owns vector t % NV of the lines t / NV, t / NV + G, ... (G = 256 / NV line groups per block); the G
// partial vectors of a block are folded in group order through shared memory
template <int RF>
__global__ void __launch_bounds__(256)
reduce_across_small_kernel(float* __restrict__ dst, const float* __restrict__ src, int n_contig, int n_strided,
                           float fnew, float fold, int nsplit, float* __restrict__ pval, int* __restrict__ pidx) {
    using F = Fn<RF>;
    __shared__ float s_val[1024];
    __shared__ int s_idx[1024];
    const int nv = n_contig >> 2, groups = 256 / nv;
    const int q = threadIdx.x % nv, grp = threadIdx.x / nv;
    const int z = blockIdx.x;
    const int j0 = (int)((long long)n_strided * z / nsplit), j1 = (int)((long long)n_strided * (z + 1) / nsplit);
    float val[4];
    int idx[4];
#pragma unroll
    for (int v = 0; v < 4; v++) { val[v] = F::init(); idx[v] = 0; }
    const float* p = src + 4 * q;
#pragma unroll 4
    for (int j = j0 + grp; j < j1; j += groups) {
        const float4 x = __ldg(reinterpret_cast<const float4*>(p + (size_t)j * n_contig));
        F::rv(val[0], idx[0], x.x, j); F::rv(val[1], idx[1], x.y, j);
        F::rv(val[2], idx[2], x.z, j); F::rv(val[3], idx[3], x.w, j);
    }
#pragma unroll
    for (int v = 0; v < 4; v++) { s_val[threadIdx.x * 4 + v] = val[v]; s_idx[threadIdx.x * 4 + v] = idx[v]; }
    __syncthreads();
    if (threadIdx.x < n_contig) {
        const int o = threadIdx.x;
        // words of output o: group g holds it at ((g*nv + o/4)*4 + o%4) = g*n_contig + o
        float r = s_val[o];
        int ri = s_idx[o];
        for (int g = 1; g < groups; g++) F::rr(r, ri, s_val[g * n_contig + o], s_idx[g * n_contig + o]);
        if (nsplit == 1) F::finish(dst + o, r, ri, fnew, fold, (float)n_strided);
        else {
            pval[(size_t)z * n_contig + o] = r;
            if (F::is_arg) pidx[(size_t)z * n_contig + o] = ri;
        }
    }
}

template <int RF>
static int launch_reduce_t(float* dst, const float* src, long long n_contig, long long n_strided, bool over_strided,
                           float fnew, float fold, cudaStream_t st) {
    const int sms = sm_count();
    const bool vec = (n_contig % 4 == 0) && ((reinterpret_cast<uintptr_t>(src) & 15) == 0);
    int rc;
    if (over_strided && vec && n_contig <= 256 && ((n_contig >> 2) & ((n_contig >> 2) - 1)) == 0 && n_strided >= 4096) {
        // few outputs, many lines: blocks split the lines, every thread of a block reads
        int nsplit = (int)std::min<long long>(8LL * sms, n_strided / 1024);
        nsplit = std::max(1, nsplit);
        float* pval = nullptr; int* pidx = nullptr;
        if (nsplit > 1) {
            void* ws;
            rc = get_workspace(st, (size_t)nsplit * n_contig * 8, &ws);
            if (rc) return rc;
            pval = (float*)ws; pidx = (int*)(pval + (size_t)nsplit * n_contig);
        }
        reduce_across_small_kernel<RF><<<nsplit, 256, 0, st>>>(dst, src, (int)n_contig, (int)n_strided, fnew, fold, nsplit, pval, pidx);
        count_launch();
        rc = check_launch("reduce_across_small_kernel");
        if (rc) return rc;
        if (nsplit > 1) {
            reduce_combine_kernel<RF><<<(unsigned)((n_contig + 255) / 256), 256, 0, st>>>(dst, n_contig, fnew, fold, nsplit, pval, pidx, (float)n_strided);
            count_launch();
            rc = check_launch("reduce_combine_kernel");
        }
        return rc;
    }
    if (over_strided) {
        const long long per_block = (long long)RA_THREADS * (vec ? 4 : 1);
        const long long gx = (n_contig + per_block - 1) / per_block;
        int nsplit = 1;
        if (gx < 4LL * sms) nsplit = (int)std::min<long long>((4LL * sms + gx - 1) / gx, std::max<long long>(1, n_strided / 16));
        nsplit = std::max(1, std::min(nsplit, 1024));
        float* pval = nullptr; int* pidx = nullptr;
        if (nsplit > 1) {
            void* ws;
            rc = get_workspace(st, (size_t)nsplit * n_contig * 8, &ws);
            if (rc) return rc;
            pval = (float*)ws; pidx = (int*)(pval + (size_t)nsplit * n_contig);
        }
        dim3 grid((unsigned)gx, nsplit);
        if (vec) reduce_across_kernel<RF, 4><<<grid, RA_THREADS, 0, st>>>(dst, src, n_contig, (int)n_strided, fnew, fold, nsplit, pval, pidx);
        else     reduce_across_kernel<RF, 1><<<grid, RA_THREADS, 0, st>>>(dst, src, n_contig, (int)n_strided, fnew, fold, nsplit, pval, pidx);
        count_launch();
        rc = check_launch("reduce_across_kernel");
        if (rc) return rc;
        if (nsplit > 1) {
            reduce_combine_kernel<RF><<<(unsigned)((n_contig + 255) / 256), 256, 0, st>>>(dst, n_contig, fnew, fold, nsplit, pval, pidx, (float)n_strided);
            count_launch();
            rc = check_launch("reduce_combine_kernel");
        }
        return rc;
    }
    if (vec && n_contig <= 64 && n_strided >= 2LL * sms) {
        // lines of at most 16 vectors: 2, 4 or 8 lanes per line
        const int lpl = n_contig <= 16 ? 2 : n_contig <= 32 ? 4 : 8;
        const long long lines_per_block = 8LL * (32 / lpl);
        const unsigned gx = (unsigned)((n_strided + lines_per_block - 1) / lines_per_block);
        if (lpl == 2) reduce_along_subwarp_kernel<RF, 4, 2><<<gx, 256, 0, st>>>(dst, src, n_contig, (int)n_strided, fnew, fold);
        else if (lpl == 4) reduce_along_subwarp_kernel<RF, 4, 4><<<gx, 256, 0, st>>>(dst, src, n_contig, (int)n_strided, fnew, fold);
        else reduce_along_subwarp_kernel<RF, 4, 8><<<gx, 256, 0, st>>>(dst, src, n_contig, (int)n_strided, fnew, fold);
        count_launch();
        return check_launch("reduce_along_subwarp_kernel");
    }
    if (n_contig <= 4096 && n_strided >= 2LL * sms) {
        const unsigned gx = (unsigned)((n_strided + 7) / 8);
        if (vec) reduce_along_warp_kernel<RF, 4><<<gx, 256, 0, st>>>(dst, src, n_contig, (int)n_strided, fnew, fold);
        else     reduce_along_warp_kernel<RF, 1><<<gx, 256, 0, st>>>(dst, src, n_contig, (int)n_strided, fnew, fold);
        count_launch();
        return check_launch("reduce_along_warp_kernel");
    }
    if (n_strided > 65535) { set_last_error("reduce along lines: more than 65535 long lines"); return CUVDIA_ERR_UNSUPPORTED; }
    int nsplit = 1;
    if (n_strided < 4LL * sms) nsplit = (int)std::min<long long>((4LL * sms + n_strided - 1) / n_strided, std::max<long long>(1, n_contig / 4096));
    nsplit = std::max(1, std::min(nsplit, 4096));
    float* pval = nullptr; int* pidx = nullptr;
    if (nsplit > 1) {
        void* ws;
        rc = get_workspace(st, (size_t)nsplit * n_strided * 8, &ws);
        if (rc) return rc;
        pval = (float*)ws; pidx = (int*)(pval + (size_t)nsplit * n_strided);
    }
    dim3 grid(nsplit, (unsigned)n_strided);
    if (vec) reduce_along_block_kernel<RF, 4><<<grid, 256, 0, st>>>(dst, src, n_contig, (int)n_strided, fnew, fold, nsplit, pval, pidx);
    else     reduce_along_block_kernel<RF, 1><<<grid, 256, 0, st>>>(dst, src, n_contig, (int)n_strided, fnew, fold, nsplit, pval, pidx);
    count_launch();
    rc = check_launch("reduce_along_block_kernel");
    if (rc) return rc;
    if (nsplit > 1) {
        reduce_combine_kernel<RF><<<(unsigned)((n_strided + 255) / 256), 256, 0, st>>>(dst, n_strided, fnew, fold, nsplit, pval, pidx, (float)n_contig);
        count_launch();
        rc = check_launch("reduce_combine_kernel");
    }
    return rc;
}

// ------------------------------------------------------------------------------------------------
// Allocation-free variant (cuvdia_reduce_noalloc_f32).
//
// The split reductions above need a scratch buffer for the per-block partial results and get it
// from the per-stream workspace, which is created with cudaMalloc on first use.  Some callers must
// not allocate: code running inside a fixed device-memory budget handed out by a host application,
// real-time or long-running services that forbid allocator calls after start-up (an allocation can
// synchronise the whole device), and code that has no way to free what a library allocated behind
// its back.  For them the partial results live in the array below, which is part of the library
// image: every device that loads the library holds these bytes until the process exits.
//
// In host code `g_noalloc_scratch` only names the symbol; it is NOT a device address, and a kernel
// handed that host-side name would fault or silently use the wrong memory.  The device address is
// looked up once per device with cudaGetSymbolAddress while that device is current, and that
// pointer is what the kernels receive.
// ------------------------------------------------------------------------------------------------
constexpr size_t NOALLOC_SCRATCH_BYTES = (size_t)4 << 20;      // 4 MiB per device
static __device__ __align__(256) unsigned char g_noalloc_scratch[NOALLOC_SCRATCH_BYTES];

// Device address of the static scratch on the current device (looked up on the first call per device).
static int noalloc_scratch_ptr(void** out) {
    // two host threads may make the first call on a device at once: both look the address up and store the same value
    static std::atomic<void*> cached[64];
    int dev = 0;
    CUVDIA_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) { set_last_error("device index %d out of range", dev); return CUVDIA_ERR_UNSUPPORTED; }
    void* p = cached[dev].load(std::memory_order_acquire);
    if (!p) {
        cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
        if (e != cudaSuccess) return cuda_fail(e, "cudaGetSymbolAddress(g_noalloc_scratch)");
        cached[dev].store(p, std::memory_order_release);
    }
    *out = p;
    return CUVDIA_OK;
}

template <int RF>
static int launch_reduce_noalloc_t(float* dst, const float* src, long long n_contig, long long n_strided,
                                   bool over_strided, float fnew, float fold, cudaStream_t st) {
    const int sms = sm_count();
    const bool vec = (n_contig % 4 == 0) && ((reinterpret_cast<uintptr_t>(src) & 15) == 0);
    const long long n_out = over_strided ? n_contig : n_strided;
    const long long n_red = over_strided ? n_strided : n_contig;
    // same split heuristics as the allocating entry point
    int nsplit = 1;
    long long gx = 0;
    if (over_strided) {
        const long long per_block = (long long)RA_THREADS * (vec ? 4 : 1);
        gx = (n_contig + per_block - 1) / per_block;
        if (gx < 4LL * sms) nsplit = (int)std::min<long long>((4LL * sms + gx - 1) / gx, std::max<long long>(1, n_strided / 16));
        nsplit = std::max(1, std::min(nsplit, 1024));
    } else {
        if (n_contig <= 4096 && n_strided >= 2LL * sms) {       // a warp per line: no scratch at all
            const unsigned g = (unsigned)((n_strided + 7) / 8);
            if (vec) reduce_along_warp_kernel<RF, 4><<<g, 256, 0, st>>>(dst, src, n_contig, (int)n_strided, fnew, fold);
            else     reduce_along_warp_kernel<RF, 1><<<g, 256, 0, st>>>(dst, src, n_contig, (int)n_strided, fnew, fold);
            count_launch();
            return check_launch("reduce_along_warp_kernel");
        }
        if (n_strided > 65535) { set_last_error("reduce along lines: more than 65535 long lines"); return CUVDIA_ERR_UNSUPPORTED; }
        if (n_strided < 4LL * sms) nsplit = (int)std::min<long long>((4LL * sms + n_strided - 1) / n_strided, std::max<long long>(1, n_contig / 4096));
        nsplit = std::max(1, std::min(nsplit, 4096));
    }
    float* pval = nullptr; int* pidx = nullptr;
    if (nsplit > 1) {
        const size_t need = (size_t)nsplit * (size_t)n_out * 8;
        if (need > NOALLOC_SCRATCH_BYTES) {
            set_last_error("cuvdia_reduce_noalloc_f32: this shape needs %zu bytes of scratch (%d partial results for each "
                           "of %lld outputs) but the static scratch holds %zu bytes; use cuvdia_reduce_f32",
                           need, nsplit, n_out, NOALLOC_SCRATCH_BYTES);
            return CUVDIA_ERR_UNSUPPORTED;
        }
        void* ws = nullptr;
        int rc = noalloc_scratch_ptr(&ws);
        if (rc) return rc;
        // every partial slot that the second stage reads is written by the first stage of the same
        // call, so nothing has to be cleared even though the array keeps the previous call's contents
        pval = (float*)ws; pidx = (int*)(pval + (size_t)nsplit * n_out);
    }
    int rc;
    if (over_strided) {
        dim3 grid((unsigned)gx, nsplit);
        if (vec) reduce_across_kernel<RF, 4><<<grid, RA_THREADS, 0, st>>>(dst, src, n_contig, (int)n_strided, fnew, fold, nsplit, pval, pidx);
        else     reduce_across_kernel<RF, 1><<<grid, RA_THREADS, 0, st>>>(dst, src, n_contig, (int)n_strided, fnew, fold, nsplit, pval, pidx);
        count_launch();
        rc = check_launch("reduce_across_kernel");
    } else {
        dim3 grid(nsplit, (unsigned)n_strided);
        if (vec) reduce_along_block_kernel<RF, 4><<<grid, 256, 0, st>>>(dst, src, n_contig, (int)n_strided, fnew, fold, nsplit, pval, pidx);
        else     reduce_along_block_kernel<RF, 1><<<grid, 256, 0, st>>>(dst, src, n_contig, (int)n_strided, fnew, fold, nsplit, pval, pidx);
        count_launch();
        rc = check_launch("reduce_along_block_kernel");
    }
    if (rc) return rc;
    if (nsplit > 1) {
        reduce_combine_kernel<RF><<<(unsigned)((n_out + 255) / 256), 256, 0, st>>>(dst, n_out, fnew, fold, nsplit, pval, pidx, (float)n_red);
        count_launch();
        rc = check_launch("reduce_combine_kernel");
    }
    return rc;
}

int launch_reduce_noalloc(float* dst, const float* src, long long n_contig, long long n_strided, bool over_strided,
                          int functor, float fnew, float fold, cudaStream_t st) {
#define CASE(RF) case RF: return launch_reduce_noalloc_t<RF>(dst, src, n_contig, n_strided, over_strided, fnew, fold, st)
    switch (functor) {
        CASE(CUVDIA_RF_ADD); CASE(CUVDIA_RF_MEAN); CASE(CUVDIA_RF_ADD_SQUARED); CASE(CUVDIA_RF_MAX);
        CASE(CUVDIA_RF_ARGMAX); CASE(CUVDIA_RF_ARGMIN); CASE(CUVDIA_RF_MIN); CASE(CUVDIA_RF_MULT);
        CASE(CUVDIA_RF_LOGADDEXP); CASE(CUVDIA_RF_ADDEXP);
    }
#undef CASE
    set_last_error("unknown reduce functor %d", functor);
    return CUVDIA_ERR_INVALID;
}

// Second stage alone, for kernels elsewhere in the library that produce per-slab partial sums themselves.
int launch_reduce_combine_add(float* dst, long long n_out, float fnew, float fold, int nsplit, const float* partial,
                              cudaStream_t st) {
    reduce_combine_kernel<CUVDIA_RF_ADD><<<(unsigned)((n_out + 255) / 256), 256, 0, st>>>(dst, n_out, fnew, fold, nsplit,
                                                                                           partial, nullptr, 1.f);
    count_launch();
    return check_launch("reduce_combine_kernel");
}

int launch_reduce(float* dst, const float* src, long long n_contig, long long n_strided, bool over_strided,
                  int functor, float fnew, float fold, cudaStream_t st) {
#define CASE(RF) case RF: return launch_reduce_t<RF>(dst, src, n_contig, n_strided, over_strided, fnew, fold, st)
    switch (functor) {
        CASE(CUVDIA_RF_ADD); CASE(CUVDIA_RF_MEAN); CASE(CUVDIA_RF_ADD_SQUARED); CASE(CUVDIA_RF_MAX);
        CASE(CUVDIA_RF_ARGMAX); CASE(CUVDIA_RF_ARGMIN); CASE(CUVDIA_RF_MIN); CASE(CUVDIA_RF_MULT);
        CASE(CUVDIA_RF_LOGADDEXP); CASE(CUVDIA_RF_ADDEXP);
    }
#undef CASE
    set_last_error("unknown reduce functor %d", functor);
    return CUVDIA_ERR_INVALID;
}

}  // namespace cuvdia

// The allocation-free entry point is defined beside its scratch array (see the block comment above
// g_noalloc_scratch).
extern "C" int cuvdia_reduce_noalloc_f32(float* dst, const float* src, long long n_contig, long long n_strided,
                                         int over_strided, int functor, float factNew, float factOld, void* stream) {
    CUVDIA_REQUIRE(dst != nullptr);
    CUVDIA_REQUIRE(src != nullptr);
    CUVDIA_REQUIRE(n_contig > 0 && n_strided > 0);
    CUVDIA_REQUIRE(n_contig * n_strided <= 2147483647LL);
    CUVDIA_REQUIRE(functor >= CUVDIA_RF_ADD && functor <= CUVDIA_RF_ADDEXP);
    if (functor == CUVDIA_RF_MEAN) {
        CUVDIA_REQUIRE(factNew == 1.f);
        CUVDIA_REQUIRE(factOld == 0.f);
    }
    return cuvdia::launch_reduce_noalloc(dst, src, n_contig, n_strided, over_strided != 0, functor, factNew, factOld,
                                         (cudaStream_t)stream);
}
