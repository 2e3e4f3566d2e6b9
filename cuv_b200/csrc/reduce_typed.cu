// reduce_to_col / reduce_to_row between element types other than float -> float.
//
// CUV instantiates nine (source, destination) pairs over float, int, unsigned int and unsigned char
// (matrix_ops/matrix_ops_reduce.cu:382-413).  Its host and device code keep the running value in the SOURCE
// type (reduce_impl::reduce, :217-292; kernels :39-147) and fold one element with a functor that computes
// in the DESTINATION type (reduce_switch, :304-343):
//     ADD / MEAN      r = (S)((D)r + (D)x)                 bf_plus<D,D,S>          (tensor_ops/functors.hpp:374)
//     ADD_SQUARED     r = (S)((D)r + (D)(x*x))             bf_add_square<D,D,S>    (:392)
//     MAX / MIN       r = r > x ? r : x  (in S)            bf_max / bf_min<S,S,S>  (:401-404)
//     ARGMAX / ARGMIN first index of the extreme (in S)    reduce_argmax / argmin  (:574-592)
// and finish with  dst = factNew*r  or  dst = factOld*dst + factNew*r,  the factors being of type S and the
// expression following C++'s usual arithmetic conversions before it is stored as D (:277-283); the index
// functors store the index; MEAN then divides by the line length in D (:312).
//
// For integer types every step above is integer arithmetic that wraps to the width of S (int, unsigned: 32 bits;
// unsigned char: 8 bits; through float it is exact while the running sums stay below 2^24), so the result does
// not depend on the order of the fold and the kernels here may sum in parallel: they add the converted elements in
// 64-bit integers, narrow once at the end, and are bit-identical to the sequential host loop wherever C++ defines
// that loop's conversions (no float -> integer conversion out of range, no signed overflow).  The comparisons of
// MAX / MIN / ARG* are exact in any order (ties go to the lowest index, as in a sequential scan).
// The logarithmic functors (MULT, LOGADDEXP, ADDEXP) are offered for float -> float only.
#include <cfloat>
#include <climits>
#include <type_traits>

#include "cuvdia_internal.cuh"

namespace cuvdia {

typedef unsigned char uchar;

template <class T> struct Lim;
template <> struct Lim<float> { __host__ __device__ static float lo() { return -FLT_MAX; } __host__ __device__ static float hi() { return FLT_MAX; } };
template <> struct Lim<int> { __host__ __device__ static int lo() { return INT_MIN; } __host__ __device__ static int hi() { return INT_MAX; } };
template <> struct Lim<unsigned> { __host__ __device__ static unsigned lo() { return 0u; } __host__ __device__ static unsigned hi() { return UINT_MAX; } };
template <> struct Lim<uchar> { __host__ __device__ static uchar lo() { return 0; } __host__ __device__ static uchar hi() { return 255; } };

// what one element contributes to the integer sum: the value the fold adds, (D)x or (D)(x*x)
template <class S, class D, bool SQ>
__device__ __forceinline__ long long contribution(S x) {
    if (SQ) return (long long)(D)(x * x);       // x*x in S's promoted arithmetic, as in bf_add_square
    return (long long)(D)x;
}
// the running value after the fold, narrowed to S as the reference stores it
template <class S, class D>
__device__ __forceinline__ S narrow(long long sum) {
    if (sizeof(D) == 1 || sizeof(S) == 1) return (S)(uchar)(unsigned long long)sum;     // 8-bit wrap on either side
    if (!std::is_floating_point<S>::value) return (S)(unsigned)(unsigned long long)sum; // S is int or unsigned: 32-bit wrap
    // S is float, D is int or unsigned: the sum lives in D between steps
    return (S)(D)(unsigned)(unsigned long long)sum;
}

template <class S, class D>
__device__ __forceinline__ void finish_typed(D* dst, S r, float fnew_f, float fold_f, int mean, long long n_red) {
    const S fnew = (S)fnew_f, fold = (S)fold_f;
    D out;
    if (fold != 0) out = fold * *dst + fnew * r;          // usual arithmetic conversions, then stored as D
    else out = fnew * r;
    if (mean) out = out / (D)n_red;
    *dst = out;
}

enum { OP_SUM = 0, OP_SUMSQ, OP_MAX, OP_MIN, OP_ARGMAX, OP_ARGMIN };

// across lines: one thread per output (contiguous position), blockIdx.y takes a share of the lines
template <class S, class D, int OP>
__global__ void __launch_bounds__(256)
reduce_across_typed_kernel(D* __restrict__ dst, const S* __restrict__ src, long long n_contig, int n_strided, float fnew,
                           float fold, int mean, int nsplit, long long* __restrict__ psum, int* __restrict__ pidx) {
    const long long o = (long long)blockIdx.x * 256 + threadIdx.x;
    if (o >= n_contig) return;
    const int z = blockIdx.y;
    const int j0 = (int)((long long)n_strided * z / nsplit), j1 = (int)((long long)n_strided * (z + 1) / nsplit);
    long long sum = 0;
    S ext = (OP == OP_MAX || OP == OP_ARGMAX) ? Lim<S>::lo() : Lim<S>::hi();
    int idx = 0;
#pragma unroll 4
    for (int j = j0; j < j1; j++) {
        const S x = src[(size_t)j * n_contig + o];
        if (OP == OP_SUM) sum += contribution<S, D, false>(x);
        else if (OP == OP_SUMSQ) sum += contribution<S, D, true>(x);
        else if (OP == OP_MAX) ext = ext > x ? ext : x;
        else if (OP == OP_MIN) ext = ext < x ? ext : x;
        else if (OP == OP_ARGMAX) { if (x > ext) { ext = x; idx = j; } }
        else { if (x < ext) { ext = x; idx = j; } }
    }
    if (nsplit > 1) {
        // partial results: the sum, or the extreme value widened to 64 bits (bit pattern for float) and its index
        long long p;
        if (OP <= OP_SUMSQ) p = sum;
        else if (std::is_floating_point<S>::value) p = (long long)__float_as_int((float)ext);
        else p = (long long)ext;
        psum[(size_t)z * n_contig + o] = p;
        if (OP >= OP_ARGMAX) pidx[(size_t)z * n_contig + o] = idx;
        return;
    }
    if (OP >= OP_ARGMAX) dst[o] = (D)(unsigned)idx;
    else finish_typed<S, D>(dst + o, OP <= OP_SUMSQ ? narrow<S, D>(sum) : ext, fnew, fold, mean, n_strided);
}

template <class S, class D, int OP>
__global__ void __launch_bounds__(256)
reduce_combine_typed_kernel(D* __restrict__ dst, long long n_out, float fnew, float fold, int mean, long long n_red,
                            int nsplit, const long long* __restrict__ psum, const int* __restrict__ pidx) {
    const long long o = (long long)blockIdx.x * 256 + threadIdx.x;
    if (o >= n_out) return;
    auto unpack = [](long long p) -> S {
        if (std::is_floating_point<S>::value) return (S)__int_as_float((int)p);
        return (S)p;
    };
    long long sum = psum[o];
    S ext = unpack(sum);
    int idx = OP >= OP_ARGMAX ? pidx[o] : 0;
    for (int z = 1; z < nsplit; z++) {
        const long long p = psum[(size_t)z * n_out + o];
        if (OP <= OP_SUMSQ) sum += p;
        else {
            const S x = unpack(p);
            if (OP == OP_MAX) ext = ext > x ? ext : x;
            else if (OP == OP_MIN) ext = ext < x ? ext : x;
            else if (OP == OP_ARGMAX) { if (x > ext) { ext = x; idx = pidx[(size_t)z * n_out + o]; } }    // later shares hold later indices
            else { if (x < ext) { ext = x; idx = pidx[(size_t)z * n_out + o]; } }
        }
    }
    if (OP >= OP_ARGMAX) dst[o] = (D)(unsigned)idx;
    else finish_typed<S, D>(dst + o, OP <= OP_SUMSQ ? narrow<S, D>(sum) : ext, fnew, fold, mean, n_red);
}

// along lines: a warp per line
template <class S, class D, int OP>
__global__ void __launch_bounds__(256)
reduce_along_typed_kernel(D* __restrict__ dst, const S* __restrict__ src, long long n_contig, long long n_strided, float fnew,
                          float fold, int mean) {
    const int lane = threadIdx.x & 31;
    const long long line = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (line >= n_strided) return;
    const S* p = src + line * n_contig;
    long long sum = 0;
    S ext = (OP == OP_MAX || OP == OP_ARGMAX) ? Lim<S>::lo() : Lim<S>::hi();
    int idx = 0;
    for (long long j = lane; j < n_contig; j += 32) {
        const S x = p[j];
        if (OP == OP_SUM) sum += contribution<S, D, false>(x);
        else if (OP == OP_SUMSQ) sum += contribution<S, D, true>(x);
        else if (OP == OP_MAX) ext = ext > x ? ext : x;
        else if (OP == OP_MIN) ext = ext < x ? ext : x;
        else if (OP == OP_ARGMAX) { if (x > ext) { ext = x; idx = (int)j; } }
        else { if (x < ext) { ext = x; idx = (int)j; } }
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) {
        if (OP <= OP_SUMSQ) sum += __shfl_down_sync(0xffffffffu, sum, d);
        else {
            // widen to 32 bits for the shuffle (unsigned char has no shuffle of its own)
            S x;
            if (sizeof(S) == 1) x = (S)__shfl_down_sync(0xffffffffu, (int)ext, d);
            else x = __shfl_down_sync(0xffffffffu, ext, d);
            const int i2 = __shfl_down_sync(0xffffffffu, idx, d);
            if (OP == OP_MAX) ext = ext > x ? ext : x;
            else if (OP == OP_MIN) ext = ext < x ? ext : x;
            else if (OP == OP_ARGMAX) { if (x > ext || (x == ext && i2 < idx)) { ext = x; idx = i2; } }
            else { if (x < ext || (x == ext && i2 < idx)) { ext = x; idx = i2; } }
        }
    }
    if (lane != 0) return;
    if (OP >= OP_ARGMAX) dst[line] = (D)(unsigned)idx;
    else finish_typed<S, D>(dst + line, OP <= OP_SUMSQ ? narrow<S, D>(sum) : ext, fnew, fold, mean, n_contig);
}

template <class S, class D, int OP>
static int launch_typed_op(D* dst, const S* src, long long n_contig, long long n_strided, bool over_strided, float fnew,
                           float fold, int mean, cudaStream_t st) {
    int rc;
    if (!over_strided) {
        reduce_along_typed_kernel<S, D, OP><<<(unsigned)((n_strided + 7) / 8), 256, 0, st>>>(dst, src, n_contig, n_strided,
                                                                                           fnew, fold, mean);
        count_launch();
        return check_launch("reduce_along_typed_kernel");
    }
    const long long gx = (n_contig + 255) / 256;
    int nsplit = 1;
    if (gx < 4LL * sm_count()) nsplit = (int)std::min<long long>((4LL * sm_count() + gx - 1) / gx, std::max<long long>(1, n_strided / 16));
    nsplit = std::max(1, std::min(nsplit, 1024));
    long long* psum = nullptr; int* pidx = nullptr;
    if (nsplit > 1) {
        void* ws;
        rc = get_workspace(st, (size_t)nsplit * n_contig * 12, &ws);
        if (rc) return rc;
        psum = (long long*)ws; pidx = (int*)(psum + (size_t)nsplit * n_contig);
    }
    reduce_across_typed_kernel<S, D, OP><<<dim3((unsigned)gx, nsplit), 256, 0, st>>>(dst, src, n_contig, (int)n_strided, fnew,
                                                                                     fold, mean, nsplit, psum, pidx);
    count_launch();
    rc = check_launch("reduce_across_typed_kernel");
    if (rc || nsplit == 1) return rc;
    reduce_combine_typed_kernel<S, D, OP><<<(unsigned)((n_contig + 255) / 256), 256, 0, st>>>(dst, n_contig, fnew, fold, mean,
                                                                                               n_strided, nsplit, psum, pidx);
    count_launch();
    return check_launch("reduce_combine_typed_kernel");
}

template <class S, class D>
static int launch_typed(void* dst, const void* src, long long n_contig, long long n_strided, bool over_strided, int functor,
                        float fnew, float fold, cudaStream_t st) {
    D* d = (D*)dst; const S* s = (const S*)src;
    switch (functor) {
        case CUVDIA_RF_ADD: return launch_typed_op<S, D, OP_SUM>(d, s, n_contig, n_strided, over_strided, fnew, fold, 0, st);
        case CUVDIA_RF_MEAN: return launch_typed_op<S, D, OP_SUM>(d, s, n_contig, n_strided, over_strided, fnew, fold, 1, st);
        case CUVDIA_RF_ADD_SQUARED: return launch_typed_op<S, D, OP_SUMSQ>(d, s, n_contig, n_strided, over_strided, fnew, fold, 0, st);
        case CUVDIA_RF_MAX: return launch_typed_op<S, D, OP_MAX>(d, s, n_contig, n_strided, over_strided, fnew, fold, 0, st);
        case CUVDIA_RF_MIN: return launch_typed_op<S, D, OP_MIN>(d, s, n_contig, n_strided, over_strided, fnew, fold, 0, st);
        case CUVDIA_RF_ARGMAX: return launch_typed_op<S, D, OP_ARGMAX>(d, s, n_contig, n_strided, over_strided, fnew, fold, 0, st);
        case CUVDIA_RF_ARGMIN: return launch_typed_op<S, D, OP_ARGMIN>(d, s, n_contig, n_strided, over_strided, fnew, fold, 0, st);
    }
    set_last_error("reduce functor %d is implemented for float -> float only (MULT, LOGADDEXP, ADDEXP)", functor);
    return CUVDIA_ERR_UNSUPPORTED;
}

int launch_reduce_typed(void* dst, int dst_type, const void* src, int src_type, long long n_contig, long long n_strided,
                        bool over_strided, int functor, float fnew, float fold, cudaStream_t st) {
#define PAIR(ST, DT, S, D) if (src_type == ST && dst_type == DT) \
        return launch_typed<S, D>(dst, src, n_contig, n_strided, over_strided, functor, fnew, fold, st)
    PAIR(CUVDIA_T_I32, CUVDIA_T_F32, int, float);
    PAIR(CUVDIA_T_U32, CUVDIA_T_F32, unsigned, float);
    PAIR(CUVDIA_T_U8, CUVDIA_T_F32, uchar, float);
    PAIR(CUVDIA_T_F32, CUVDIA_T_I32, float, int);
    PAIR(CUVDIA_T_F32, CUVDIA_T_U32, float, unsigned);
    PAIR(CUVDIA_T_F32, CUVDIA_T_U8, float, uchar);
    PAIR(CUVDIA_T_U8, CUVDIA_T_U8, uchar, uchar);
    PAIR(CUVDIA_T_U8, CUVDIA_T_U32, uchar, unsigned);
#undef PAIR
    set_last_error("reduce: CUV has no instantiation for source type %d and destination type %d "
                   "(matrix_ops/matrix_ops_reduce.cu:395-413)", src_type, dst_type);
    return CUVDIA_ERR_UNSUPPORTED;
}

}  // namespace cuvdia
