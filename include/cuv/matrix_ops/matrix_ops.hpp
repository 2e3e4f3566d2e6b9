// prod / spmv with a DIA operand and reduce_to_col / reduce_to_row of the CUV surface
// (matrix_ops/matrix_ops.hpp:118-119,185-228,277-278 in CUV).  The dev_memory_space versions
// forward to the cuvdia C ABI and then synchronise, because every CUV operation is blocking
// (matrix_ops/spmv.cu:99, matrix_ops_reduce.cu:186,214).  The host_memory_space versions are
// declared only: CUV's own host code is the parity reference and is not part of this library
// (the test suite links a restatement of it).
#pragma once
#include <type_traits>

#include "cuv/basics/dia_matrix.hpp"
#include "cuv/basics/tensor.hpp"

namespace cuv {

enum reduce_functor {          // matrix_ops/matrix_ops.hpp:185-196
    RF_ADD, RF_MEAN, RF_ADD_SQUARED, RF_MAX, RF_ARGMAX, RF_ARGMIN, RF_MIN, RF_MULT, RF_LOGADDEXP, RF_ADDEXP
};

// Arithmetic of the device prod: CUVDIA_MODE_EXACT (default, bit-identical to the host code) or
// CUVDIA_MODE_FAST (fused multiply-add).  Process-wide switch; CUV's signature has no room for it.
inline int& dia_prod_mode() { static int mode = CUVDIA_MODE_EXACT; return mode; }

// ---- prod(C, A_dia, B, transA, transB, factAB, factC) -------------------------------------------------
template <class V, class M, class L>
void prod(tensor<V, M, L>& C, const dia_matrix<V, M>& A, const tensor<V, M, L>& B, char transA = 'n', char transB = 'n',
          const float& factAB = 1.f, const float& factC = 0.f);

template <>
void prod(tensor<float, host_memory_space, column_major>& C, const dia_matrix<float, host_memory_space>& A,
          const tensor<float, host_memory_space, column_major>& B, char transA, char transB, const float& factAB,
          const float& factC);        // defined by the reference host code, not by this library

template <>
inline void prod(tensor<float, dev_memory_space, column_major>& C, const dia_matrix<float, dev_memory_space>& A,
                 const tensor<float, dev_memory_space, column_major>& B, char transA, char transB,
                 const float& factAB, const float& factC) {
    cuvAssert(C.shape().size() == 2);                    // matrix_ops/spmv.cu:229-232
    cuvAssert(B.shape().size() == 2);
    cuvAssert(C.shape()[1] == B.shape()[1]);
    cuvAssert(A.vec_ptr());
    if (transA == 't') { cuvAssert(A.w() == C.shape()[0]); cuvAssert(A.h() == B.shape()[0]); }
    else if (transA == 'n') { cuvAssert(A.h() == C.shape()[0]); cuvAssert(A.w() == B.shape()[0]); }
    cuvdia_check(cuvdia_prod_f32(A.plan(), A.vec().ptr(), B.ptr(), (int)B.shape()[0], C.ptr(), (int)C.shape()[0],
                                 (int)C.shape()[1], transA, transB, factAB, factC, dia_prod_mode(), 0));
    cuvSafeCall(cudaDeviceSynchronize());
    cuvdia_check_plan(A.plan());
}

// ---- spmv(dst, A, v, transA, factAv, factC): vectors packed column-major in 1-D tensors ------------------
template <class V, class M>
void spmv(tensor<V, M>& dst, const dia_matrix<V, M>& A, const tensor<V, M>& v, char transA = 'n',
          const float& factAv = 1.f, const float& factC = 0.f);

template <>
void spmv(tensor<float, host_memory_space>& dst, const dia_matrix<float, host_memory_space>& A,
          const tensor<float, host_memory_space>& v, char transA, const float& factAv, const float& factC);

template <>
inline void spmv(tensor<float, dev_memory_space>& dst, const dia_matrix<float, dev_memory_space>& A,
                 const tensor<float, dev_memory_space>& v, char transA, const float& factAv, const float& factC) {
    const unsigned rows_b = transA == 't' ? A.h() : A.w(), rows_c = transA == 't' ? A.w() : A.h();
    cuvAssert(v.size() % rows_b == 0);
    const unsigned n = v.size() / rows_b;
    cuvAssert(dst.size() == n * rows_c);
    cuvdia_check(cuvdia_prod_f32(A.plan(), A.vec().ptr(), v.ptr(), (int)rows_b, dst.ptr(), (int)rows_c, (int)n, transA,
                                 'n', factAv, factC, dia_prod_mode(), 0));
    cuvSafeCall(cudaDeviceSynchronize());
    cuvdia_check_plan(A.plan());
}

// ---- reductions ------------------------------------------------------------------------------------------
// reduce_to_col / reduce_to_row keep CUV's signature (matrix_ops/matrix_ops.hpp:211-228): destination element type V2,
// source element type V, factors of the SOURCE type.  The pairs CUV instantiates are available
// (matrix_ops/matrix_ops_reduce.cu:395-413); any other pair fails with the library's "not supported" error.
namespace detail {
template <class T> struct cuvdia_type;       // element type -> CUVDIA_T_* code
template <> struct cuvdia_type<float> { static const int code = CUVDIA_T_F32; };
template <> struct cuvdia_type<int> { static const int code = CUVDIA_T_I32; };
template <> struct cuvdia_type<unsigned int> { static const int code = CUVDIA_T_U32; };
template <> struct cuvdia_type<unsigned char> { static const int code = CUVDIA_T_U8; };

// src viewed as n_strided lines of n_contig contiguous elements.  A tensor of more than two dimensions is reduced
// like the matrix that keeps the surviving dimension and flattens the others (matrix_ops_reduce.cu:228-231,348-379):
// reduce_to_col keeps the first dimension, reduce_to_row the last.  Returns whether the reduction runs over the
// strided direction (the outputs are then the contiguous one).
template <class V, class M, class L>
inline bool reduce_dims(const tensor<V, M, L>& m, bool keep_first, long long& n_contig, long long& n_strided) {
    const bool cm = std::is_same<L, column_major>::value;
    const long long kept = keep_first ? m.shape(0) : m.shape(m.ndim() - 1), others = m.size() / kept;
    const bool kept_is_contiguous = keep_first ? cm : !cm;
    if (kept_is_contiguous) { n_contig = kept; n_strided = others; return true; }
    n_contig = others; n_strided = kept;
    return false;
}
// the reference host code (not part of this library; the test suite supplies it)
void reduce_host(void* v, int v_type, const void* m, int m_type, long long n_contig, long long n_strided,
                 bool over_strided, reduce_functor rf, float factNew, float factOld);

template <class V2, class V, class L>
inline void reduce_dev(tensor<V2, dev_memory_space>& dst, const tensor<V, dev_memory_space, L>& src, bool keep_first,
                       reduce_functor rf, const V& factNew, const V& factOld) {
    cuvAssert(src.ptr() != NULL);
    long long nc, ns;
    const bool over_strided = reduce_dims(src, keep_first, nc, ns);
    cuvAssert((long long)dst.size() == (over_strided ? nc : ns));
    cuvdia_check(cuvdia_reduce(dst.ptr(), cuvdia_type<V2>::code, src.ptr(), cuvdia_type<V>::code, nc, ns,
                               over_strided ? 1 : 0, (int)rf, (float)factNew, (float)factOld, 0));
    cuvSafeCall(cudaDeviceSynchronize());
}
template <class V2, class V, class L>
inline void reduce_hst(tensor<V2, host_memory_space>& dst, const tensor<V, host_memory_space, L>& src, bool keep_first,
                       reduce_functor rf, const V& factNew, const V& factOld) {
    long long nc, ns;
    const bool over_strided = reduce_dims(src, keep_first, nc, ns);
    cuvAssert((long long)dst.size() == (over_strided ? nc : ns));
    reduce_host(dst.ptr(), cuvdia_type<V2>::code, src.ptr(), cuvdia_type<V>::code, nc, ns, over_strided, rf,
                (float)factNew, (float)factOld);
}
}  // namespace detail

// dst[i] = factOld*dst[i] + factNew*rf_j(src(i,j)), dst.size() == src.shape(0)
template <class V2, class V, class L>
void reduce_to_col(tensor<V2, dev_memory_space>& dst, const tensor<V, dev_memory_space, L>& src, reduce_functor rf = RF_ADD,
                   const V& factNew = 1, const V& factOld = 0) {
    detail::reduce_dev(dst, src, true, rf, factNew, factOld);
}
// dst[j] = factOld*dst[j] + factNew*rf_i(src(i,j)), dst.size() == src.shape(last)
template <class V2, class V, class L>
void reduce_to_row(tensor<V2, dev_memory_space>& dst, const tensor<V, dev_memory_space, L>& src, reduce_functor rf = RF_ADD,
                   const V& factNew = 1, const V& factOld = 0) {
    detail::reduce_dev(dst, src, false, rf, factNew, factOld);
}
template <class V2, class V, class L>
void reduce_to_col(tensor<V2, host_memory_space>& dst, const tensor<V, host_memory_space, L>& src, reduce_functor rf = RF_ADD,
                   const V& factNew = 1, const V& factOld = 0) {
    detail::reduce_hst(dst, src, true, rf, factNew, factOld);
}
template <class V2, class V, class L>
void reduce_to_row(tensor<V2, host_memory_space>& dst, const tensor<V, host_memory_space, L>& src, reduce_functor rf = RF_ADD,
                   const V& factNew = 1, const V& factOld = 0) {
    detail::reduce_hst(dst, src, false, rf, factNew, factOld);
}

}  // namespace cuv
