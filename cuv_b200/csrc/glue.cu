// Element-wise glue of the RBM step: bias add + logistic + compare-to-uniform in one pass over a
// column-major activation matrix, and the AXPBY update of apply_binary_functor.
#include "cuvdia_internal.cuh"

namespace cuvdia {

__device__ __forceinline__ float sigm(float x) { return 1.f / (1.f + expf(-x)); }   // tensor_ops/functors.hpp:122

// ---- uniform numbers drawn where they are used -------------------------------------------------------------------
// CUV binarises an activation by comparing it with a uniform number drawn on the device (rnd_binarize,
// random/random.cu:86-91,139-156: one generator state per thread).  Here the number of element (row, column) of draw
// `which` in step `step` is a pure function of those four and a 64-bit seed - the counter-based generator
// Philox4x32-10 (Salmon, Moraes, Dror, Shaw: "Parallel random numbers: as easy as 1, 2, 3", SC 2011) - so a pass can
// draw it in registers instead of reading it from memory, any sharding of the batch columns draws the same numbers
// as the unsharded run, and a CPU restatement reproduces them bit for bit.  One call gives four 32-bit words: the
// numbers of rows 4q .. 4q+3 of one column; counter = (q, column, which + 65536 * (column >> 32), step), key = seed.
// A word x becomes the float (x >> 8) * 2^-24 in [0, 1): exact, and P(u < p) = p to within 2^-24.
__device__ __forceinline__ uint4 philox4x32_10(uint4 c, uint2 k) {
#pragma unroll
    for (int r = 0; r < 10; r++) {
        const unsigned long long p0 = (unsigned long long)0xD2511F53u * c.x;      // one wide multiply gives both halves
        const unsigned long long p1 = (unsigned long long)0xCD9E8D57u * c.z;
        c = make_uint4((unsigned)(p1 >> 32) ^ c.y ^ k.x, (unsigned)p1, (unsigned)(p0 >> 32) ^ c.w ^ k.y, (unsigned)p0);
        k.x += 0x9E3779B9u; k.y += 0xBB67AE85u;
    }
    return c;
}

__device__ __forceinline__ float u01(unsigned x) { return (float)(x >> 8) * (1.f / 16777216.f); }

// the four uniform numbers of rows 4q .. 4q+3 of global column gcol
__device__ __forceinline__ float4 draw4(const DrawParams& d, int q, long long gcol) {
    const uint4 r = philox4x32_10(make_uint4((unsigned)q, (unsigned)gcol, d.which + 65536u * (unsigned)(gcol >> 32), d.step),
                                  make_uint2(d.k0, d.k1));
    return make_float4(u01(r.x), u01(r.y), u01(r.z), u01(r.w));
}

__global__ void __launch_bounds__(256)
uniform_kernel(float* __restrict__ dst, int ld, int rows, int ncols, const DrawParams d) {
    const int groups = (rows + 3) / 4;
    const long long total = (long long)groups * ncols;
    for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total;
         t += (long long)gridDim.x * blockDim.x) {
        const int col = (int)(t / groups), q = (int)(t - (long long)col * groups);
        const float4 u = draw4(d, q, d.col0 + col);
        float* o = dst + (size_t)col * ld + 4 * q;
        const float v[4] = {u.x, u.y, u.z, u.w};
        for (int e = 0; e < 4 && 4 * q + e < rows; e++) o[e] = v[e];
    }
}

// act <- act > u ? 1 : 0 in place, u drawn as above (rnd_binarize, random/random.cu:86-91,139-156).
__global__ void __launch_bounds__(256)
binarize_kernel(float* __restrict__ act, int ld, int rows, int ncols, const DrawParams d) {
    const int groups = (rows + 3) / 4;
    const long long total = (long long)groups * ncols;
    for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total;
         t += (long long)gridDim.x * blockDim.x) {
        const int col = (int)(t / groups), q = (int)(t - (long long)col * groups);
        const float4 u = draw4(d, q, d.col0 + col);
        float* o = act + (size_t)col * ld + 4 * q;
        const float v[4] = {u.x, u.y, u.z, u.w};
        for (int e = 0; e < 4 && 4 * q + e < rows; e++) o[e] = o[e] > v[e] ? 1.f : 0.f;
    }
}

int launch_binarize(float* act, int ld, int rows, int ncols, const DrawParams& d, cudaStream_t st) {
    const long long total = (long long)((rows + 3) / 4) * ncols;
    const int blocks = (int)std::max<long long>(1, std::min<long long>((total + 255) / 256, 16LL * sm_count()));
    binarize_kernel<<<blocks, 256, 0, st>>>(act, ld, rows, ncols, d);
    count_launch();
    return check_launch("binarize_kernel");
}

int launch_uniform(float* dst, int ld, int rows, int ncols, const DrawParams& d, cudaStream_t st) {
    const long long total = (long long)((rows + 3) / 4) * ncols;
    const int blocks = (int)std::max<long long>(1, std::min<long long>((total + 255) / 256, 16LL * sm_count()));
    uniform_kernel<<<blocks, 256, 0, st>>>(dst, ld, rows, ncols, d);
    count_launch();
    return check_launch("uniform_kernel");
}

template <bool VEC>
__global__ void __launch_bounds__(256)
bias_sigmoid_sample_kernel(float* __restrict__ act, int ld, const float* __restrict__ bias,
                           const float* __restrict__ u, int ldu, float* __restrict__ sample, int lds,
                           int units, int ncols) {
    const int per_col = VEC ? units / 4 : units;
    const long long total = (long long)per_col * ncols;
    for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total;
         t += (long long)gridDim.x * blockDim.x) {
        const int col = (int)(t / per_col);
        const int i = (int)(t - (long long)col * per_col) * (VEC ? 4 : 1);
        if (VEC) {
            float4 a = *reinterpret_cast<float4*>(act + (size_t)col * ld + i);
            if (bias) {
                const float4 b = __ldg(reinterpret_cast<const float4*>(bias + i));
                a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
            }
            a.x = sigm(a.x); a.y = sigm(a.y); a.z = sigm(a.z); a.w = sigm(a.w);
            *reinterpret_cast<float4*>(act + (size_t)col * ld + i) = a;
            if (sample) {
                const float4 r = __ldg(reinterpret_cast<const float4*>(u + (size_t)col * ldu + i));
                float4 s;
                s.x = a.x > r.x ? 1.f : 0.f; s.y = a.y > r.y ? 1.f : 0.f;       // random/random.cu:86-91
                s.z = a.z > r.z ? 1.f : 0.f; s.w = a.w > r.w ? 1.f : 0.f;
                *reinterpret_cast<float4*>(sample + (size_t)col * lds + i) = s;
            }
        } else {
            float a = act[(size_t)col * ld + i];
            if (bias) a += bias[i];
            a = sigm(a);
            act[(size_t)col * ld + i] = a;
            if (sample) sample[(size_t)col * lds + i] = a > u[(size_t)col * ldu + i] ? 1.f : 0.f;
        }
    }
}

static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

int launch_bias_sigmoid_sample(float* act, int ld, const float* bias, const float* u, int ldu, float* sample,
                               int lds, int units, int ncols, cudaStream_t st) {
    bool vec = units % 4 == 0 && ld % 4 == 0 && aligned16(act) && (!bias || aligned16(bias));
    if (u) vec = vec && ldu % 4 == 0 && lds % 4 == 0 && aligned16(u) && aligned16(sample);
    const long long total = (long long)(vec ? units / 4 : units) * ncols;
    const int blocks = (int)std::min<long long>((total + 255) / 256, 16LL * sm_count());
    if (vec) bias_sigmoid_sample_kernel<true><<<blocks, 256, 0, st>>>(act, ld, bias, u, ldu, sample, lds, units, ncols);
    else     bias_sigmoid_sample_kernel<false><<<blocks, 256, 0, st>>>(act, ld, bias, u, ldu, sample, lds, units, ncols);
    count_launch();
    return check_launch("bias_sigmoid_sample_kernel");
}

// The same pass that also sums over the batch: a block owns 1024 (VEC) or 256 units and one slab of batch
// columns, every thread keeps the running sums of its units over the slab's columns (ascending, four columns in
// flight), and the slabs' partial sums are folded in slab order by the reductions' second stage, so the result is
// reproducible run to run.  Summed is either the activation after the logistic or the 0/1 sample; this replaces a
// separate reduce_to_col over a matrix this pass has just produced.  With store_act == 0 the activations are
// not written back (callers that only consume the sample and its sum).
// DRAW: the uniform numbers are not read from u but drawn in registers (see draw4 above).
template <bool VEC, bool DRAW>
__global__ void __launch_bounds__(256)
bias_sigmoid_sample_sum_kernel(float* __restrict__ act, int ld, const float* __restrict__ bias,
                               const float* __restrict__ u, int ldu, float* __restrict__ sample, int lds, int units,
                               int ncols, int nslab, int sum_sample, int store_act, float* __restrict__ partial,
                               float* __restrict__ dst, float fnew, float fold, const DrawParams dp) {
    constexpr int W = VEC ? 4 : 1;
    const int i = (blockIdx.x * 256 + threadIdx.x) * W;
    if (i >= units) return;
    const int z = blockIdx.y;
    const int c0 = (int)((long long)ncols * z / nslab), c1 = (int)((long long)ncols * (z + 1) / nslab);
    float bv[W], acc[W];
#pragma unroll
    for (int v = 0; v < W; v++) { bv[v] = bias ? __ldg(bias + i + v) : 0.f; acc[v] = 0.f; }
    auto one = [&](float (&a)[W], const float (&r)[W], int col) {
        float s[W];
#pragma unroll
        for (int v = 0; v < W; v++) {
            if (bias) a[v] += bv[v];
            a[v] = sigm(a[v]);
            s[v] = a[v] > r[v] ? 1.f : 0.f;                                  // random/random.cu:86-91
            acc[v] += (sum_sample ? s[v] : a[v]);
        }
        if (VEC) {
            if (store_act) *reinterpret_cast<float4*>(act + (size_t)col * ld + i) = make_float4(a[0], a[W > 1 ? 1 : 0], a[W > 2 ? 2 : 0], a[W > 3 ? 3 : 0]);
            if (sample) *reinterpret_cast<float4*>(sample + (size_t)col * lds + i) = make_float4(s[0], s[W > 1 ? 1 : 0], s[W > 2 ? 2 : 0], s[W > 3 ? 3 : 0]);
        } else {
            if (store_act) act[(size_t)col * ld + i] = a[0];
            if (sample) sample[(size_t)col * lds + i] = s[0];
        }
    };
    auto load = [&](const float* base, int pitch, int col, float (&x)[W]) {
        if (VEC) {
            const float4 t = *reinterpret_cast<const float4*>(base + (size_t)col * pitch + i);
            x[0] = t.x; x[W > 1 ? 1 : 0] = t.y; x[W > 2 ? 2 : 0] = t.z; x[W > 3 ? 3 : 0] = t.w;
        } else {
            x[0] = base[(size_t)col * pitch + i];
        }
    };
    auto draw = [&](int col, float (&x)[W]) {
        const float4 t = draw4(dp, i >> 2, dp.col0 + col);
        if (VEC) { x[0] = t.x; x[W > 1 ? 1 : 0] = t.y; x[W > 2 ? 2 : 0] = t.z; x[W > 3 ? 3 : 0] = t.w; }
        else { const int e = i & 3; x[0] = e == 0 ? t.x : e == 1 ? t.y : e == 2 ? t.z : t.w; }
    };
    int col = c0;
    for (; col + 4 <= c1; col += 4) {
        float a[4][W], r[4][W];
#pragma unroll
        for (int q = 0; q < 4; q++) {
            load(act, ld, col + q, a[q]);
            if (DRAW) draw(col + q, r[q]);
            else if (u) load(u, ldu, col + q, r[q]);
            else {
#pragma unroll
                for (int v = 0; v < W; v++) r[q][v] = 0.f;
            }
        }
#pragma unroll
        for (int q = 0; q < 4; q++) one(a[q], r[q], col + q);
    }
    for (; col < c1; col++) {
        float a[W], r[W];
        load(act, ld, col, a);
        if (DRAW) draw(col, r);
        else if (u) load(u, ldu, col, r);
        else {
#pragma unroll
            for (int v = 0; v < W; v++) r[v] = 0.f;
        }
        one(a, r, col);
    }
#pragma unroll
    for (int v = 0; v < W; v++) {
        if (nslab == 1) dst[i + v] = (fold != 0.f) ? fold * dst[i + v] + fnew * acc[v] : fnew * acc[v];
        else partial[(size_t)z * units + i + v] = acc[v];
    }
}

int launch_bias_sigmoid_sample_sum(float* act, int ld, const float* bias, const float* u, int ldu, float* sample,
                                   int lds, int units, int ncols, float* sum_dst, int sum_sample, float fnew, float fold,
                                   int store_act, cudaStream_t st, const DrawParams* draw) {
    bool vec = units % 4 == 0 && ld % 4 == 0 && aligned16(act) && (!bias || aligned16(bias));
    if (u) vec = vec && ldu % 4 == 0 && aligned16(u);
    if (sample) vec = vec && lds % 4 == 0 && aligned16(sample);
    DrawParams dp = {};
    if (draw) dp = *draw;
    const int per_block = 256 * (vec ? 4 : 1);
    const int gx = (units + per_block - 1) / per_block;
    // enough blocks to fill the device several times over, but at least 8 columns per slab
    int nslab = (int)std::min<long long>((8LL * sm_count() + gx - 1) / gx, std::max(1, ncols / 8));
    nslab = std::max(1, std::min(nslab, 1024));
    float* partial = nullptr;
    if (nslab > 1) {
        void* ws;
        int rc = get_workspace(st, (size_t)nslab * units * sizeof(float), &ws);
        if (rc) return rc;
        partial = (float*)ws;
    }
    dim3 grid(gx, nslab);
#define BSS_GO(V, D) bias_sigmoid_sample_sum_kernel<V, D><<<grid, 256, 0, st>>>(act, ld, bias, u, ldu, sample, lds, units, ncols, nslab, sum_sample, store_act, partial, sum_dst, fnew, fold, dp)
    if (draw) { if (vec) BSS_GO(true, true); else BSS_GO(false, true); }
    else      { if (vec) BSS_GO(true, false); else BSS_GO(false, false); }
#undef BSS_GO
    count_launch();
    int rc = check_launch("bias_sigmoid_sample_sum_kernel");
    if (rc || nslab == 1) return rc;
    return launch_reduce_combine_add(sum_dst, units, fnew, fold, nslab, partial, st);
}

__global__ void __launch_bounds__(256)
axpby_kernel(float* dst, const float* x, const float* y, float a, float b, long long n) {
    for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < n; t += (long long)gridDim.x * blockDim.x)
        dst[t] = a * x[t] + b * y[t];                                           // tensor_ops/functors.hpp:412-433
}

int launch_axpby(float* dst, const float* x, const float* y, float a, float b, long long n, cudaStream_t st) {
    const int blocks = (int)std::min<long long>((n + 255) / 256, 16LL * sm_count());
    axpby_kernel<<<blocks, 256, 0, st>>>(dst, x, y, a, b, n);
    count_launch();
    return check_launch("axpby_kernel");
}

// Gradient step with L2 weight decay, W = alpha*dW + beta*W with alpha = -learnrate and
// beta = 1 - learnrate*decay (tensor_ops/rprop.cu:147-156,341-346): two multiplies and an add, unfused,
// like the host loop (rprop.cu:331-339).  Four values per thread when the pointers allow.
template <bool VEC>
__global__ void __launch_bounds__(256)
learn_step_kernel(float* __restrict__ W, const float* __restrict__ dW, float alpha, float beta, long long n) {
    const long long stride = (long long)gridDim.x * blockDim.x;
    if (VEC) {
        const long long n4 = n / 4;
        for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < n4; t += stride) {
            const float4 g = __ldg(reinterpret_cast<const float4*>(dW) + t);
            float4 w = reinterpret_cast<float4*>(W)[t];
            w.x = __fadd_rn(__fmul_rn(alpha, g.x), __fmul_rn(beta, w.x));
            w.y = __fadd_rn(__fmul_rn(alpha, g.y), __fmul_rn(beta, w.y));
            w.z = __fadd_rn(__fmul_rn(alpha, g.z), __fmul_rn(beta, w.z));
            w.w = __fadd_rn(__fmul_rn(alpha, g.w), __fmul_rn(beta, w.w));
            reinterpret_cast<float4*>(W)[t] = w;
        }
        for (long long t = 4 * n4 + (long long)blockIdx.x * blockDim.x + threadIdx.x; t < n; t += stride)
            W[t] = __fadd_rn(__fmul_rn(alpha, dW[t]), __fmul_rn(beta, W[t]));
    } else {
        for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < n; t += stride)
            W[t] = __fadd_rn(__fmul_rn(alpha, dW[t]), __fmul_rn(beta, W[t]));
    }
}

// The same step with momentum (tensor_ops/rprop.cu:158-170, the device kernel's formula):
//   m = momentum_weight*m - lr*(dW + l2decay*W);  W += m;  M = m
template <bool VEC>
__global__ void __launch_bounds__(256)
learn_step_momentum_kernel(float* __restrict__ W, float* __restrict__ M, const float* __restrict__ dW, float lr,
                           float mw, float l2, long long n) {
    const long long stride = (long long)gridDim.x * blockDim.x;
    auto one = [&](float w, float m, float g, float& w_out, float& m_out) {
        m_out = __fsub_rn(__fmul_rn(mw, m), __fmul_rn(lr, __fadd_rn(g, __fmul_rn(l2, w))));
        w_out = __fadd_rn(w, m_out);
    };
    if (VEC) {
        const long long n4 = n / 4;
        for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < n4; t += stride) {
            const float4 g = __ldg(reinterpret_cast<const float4*>(dW) + t);
            float4 w = reinterpret_cast<float4*>(W)[t];
            float4 m = reinterpret_cast<float4*>(M)[t];
            one(w.x, m.x, g.x, w.x, m.x); one(w.y, m.y, g.y, w.y, m.y);
            one(w.z, m.z, g.z, w.z, m.z); one(w.w, m.w, g.w, w.w, m.w);
            reinterpret_cast<float4*>(W)[t] = w;
            reinterpret_cast<float4*>(M)[t] = m;
        }
        for (long long t = 4 * n4 + (long long)blockIdx.x * blockDim.x + threadIdx.x; t < n; t += stride)
            one(W[t], M[t], dW[t], W[t], M[t]);
    } else {
        for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < n; t += stride)
            one(W[t], M[t], dW[t], W[t], M[t]);
    }
}

int launch_learn_step(float* W, float* M, const float* dW, float a, float b, float c, long long n, cudaStream_t st) {
    const bool vec = aligned16(W) && aligned16(dW) && (!M || aligned16(M));
    const long long work = vec ? (n + 3) / 4 : n;
    const int blocks = (int)std::max<long long>(1, std::min<long long>((work + 255) / 256, 16LL * sm_count()));
    if (M) {
        if (vec) learn_step_momentum_kernel<true><<<blocks, 256, 0, st>>>(W, M, dW, a, b, c, n);
        else     learn_step_momentum_kernel<false><<<blocks, 256, 0, st>>>(W, M, dW, a, b, c, n);
    } else {
        if (vec) learn_step_kernel<true><<<blocks, 256, 0, st>>>(W, dW, a, b, n);
        else     learn_step_kernel<false><<<blocks, 256, 0, st>>>(W, dW, a, b, n);
    }
    count_launch();
    return check_launch(M ? "learn_step_momentum_kernel" : "learn_step_kernel");
}

// dst[i] = op(x[i], y[i]) with the parameterised functors of apply_binary_functor
// (tensor_ops/functors.hpp:377-433): op codes are CUVDIA_BF_*.
__global__ void __launch_bounds__(256)
binary_kernel(float* dst, const float* x, const float* y, int op, float p, float p2, long long n) {
    for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < n; t += (long long)gridDim.x * blockDim.x) {
        const float a = x[t], b = y[t];
        float r;
        switch (op) {
            case CUVDIA_BF_ADD: r = a + b; break;
            case CUVDIA_BF_SUBTRACT: r = a - b; break;
            case CUVDIA_BF_MULT: r = a * b; break;
            case CUVDIA_BF_AXPY: r = p * a + b; break;
            case CUVDIA_BF_XPBY: r = a + p * b; break;
            default: r = p * a + p2 * b; break;     // CUVDIA_BF_AXPBY
        }
        dst[t] = r;
    }
}

int launch_binary(float* dst, const float* x, const float* y, int op, float p, float p2, long long n, cudaStream_t st) {
    const int blocks = (int)std::min<long long>((n + 255) / 256, 16LL * sm_count());
    binary_kernel<<<blocks, 256, 0, st>>>(dst, x, y, op, p, p2, n);
    count_launch();
    return check_launch("binary_kernel");
}

// dst[i] = value (sequence == 0) or dst[i] = i (sequence != 0): fill / sequence of tensor_ops.hpp:108-122
__global__ void __launch_bounds__(256) fill_kernel(float* dst, float value, int sequence, long long n) {
    for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < n; t += (long long)gridDim.x * blockDim.x)
        dst[t] = sequence ? (float)t : value;
}

int launch_fill(float* dst, float value, int sequence, long long n, cudaStream_t st) {
    const int blocks = (int)std::min<long long>((n + 255) / 256, 16LL * sm_count());
    fill_kernel<<<blocks, 256, 0, st>>>(dst, value, sequence, n);
    count_launch();
    return check_launch("fill_kernel");
}

}  // namespace cuvdia
