// TEST INFRASTRUCTURE ONLY.  Supplies the host_memory_space halves of the CUV surface (prod, spmv,
// densedense_to_dia, reductions) by calling the CPU oracle (cuv_host_oracle.c), so that the C++
// tests can do what CUV's own tests do: run the same template on a host and a device object and
// compare.  The library never includes or links this file.
#pragma once
#include "cuv.hpp"

extern "C" {
int oracle_prod_dia(float* C, int ldc, const float* vals, const int* offsets, int nd, int h, int w, int stride, int rf,
                    const float* B, int ldb, int ncols, char transA, float factAB, float factC, int nthreads);
int oracle_dd2dia(float* Cvals, const int* offsets, int nd, int h, int w, int stride, int rf, const float* A, int lda,
                  const float* B, int ldb, int ncols, float factAB, float factC, int literal_host, int nthreads);
int oracle_reduce(float* dst, const float* src, long n_contig, long n_strided, int over_strided, int rf, float factNew,
                  float factOld, int nthreads);
int oracle_avg_diagonals(float* dst, const float* vals, const int* offsets, int nd, int h, int w, int stride, int rf);
int oracle_reduce_typed(void* dst, int dst_type, const void* src, int src_type, long n_contig, long n_strided,
                        int over_strided, int rf, float factNew, float factOld);
void oracle_uniform(float* dst, long ld, long rows, long ncols, unsigned long long seed, unsigned long long step,
                    long long col0, int which);
void oracle_learn_step_weight_decay(float* W, const float* dW, long n, float learnrate, float decay);
void oracle_learn_step_weight_decay_momentum(float* W, float* M, const float* dW, long n, float lr, float mw, float l2,
                                             int device_formula);
}

namespace cuv {

template <>
inline void prod(tensor<float, host_memory_space, column_major>& C, const dia_matrix<float, host_memory_space>& A,
                 const tensor<float, host_memory_space, column_major>& B, char transA, char transB, const float& factAB,
                 const float& factC) {
    cuvAssert(C.shape().size() == 2);                    // matrix_ops/spmv.cu:211-214
    cuvAssert(B.shape().size() == 2);
    cuvAssert(transB == 'n');
    cuvAssert(C.shape()[1] == B.shape()[1]);
    if (transA == 't') { cuvAssert(A.h() == B.shape()[0]); cuvAssert(A.w() == C.shape()[0]); }
    else { cuvAssert(A.w() == B.shape()[0]); cuvAssert(A.h() == C.shape()[0]); }
    cuvAssert(oracle_prod_dia(C.ptr(), C.shape()[0], A.vec().ptr(), A.get_offsets().ptr(), A.num_dia(), A.h(), A.w(),
                              A.stride(), A.row_fact(), B.ptr(), B.shape()[0], C.shape()[1], transA, factAB, factC, 1) == 0);
}

template <>
inline void spmv(tensor<float, host_memory_space>& dst, const dia_matrix<float, host_memory_space>& A,
                 const tensor<float, host_memory_space>& v, char transA, const float& factAv, const float& factC) {
    const unsigned rows_b = transA == 't' ? A.h() : A.w(), rows_c = transA == 't' ? A.w() : A.h();
    cuvAssert(oracle_prod_dia(dst.ptr(), rows_c, A.vec().ptr(), A.get_offsets().ptr(), A.num_dia(), A.h(), A.w(),
                              A.stride(), A.row_fact(), v.ptr(), rows_b, v.size() / rows_b, transA, factAv, factC, 1) == 0);
}

template <class V, class L, class I>
void densedense_to_dia(dia_matrix<V, host_memory_space, I>& C, const host_block_descriptor<V, I>&,
                       const tensor<V, host_memory_space, L>& A, const tensor<V, host_memory_space, L>& B,
                       const V& factAB, const V& factC) {
    cuvAssert(C.w() == B.shape()[0]);                    // matrix_ops/densedense_to_sparse.cu:214-216
    cuvAssert(C.h() == A.shape()[0]);
    cuvAssert(A.shape()[1] == B.shape()[1]);
    cuvAssert(oracle_dd2dia(C.vec().ptr(), C.get_offsets().ptr(), C.num_dia(), C.h(), C.w(), C.stride(), C.row_fact(),
                            A.ptr(), A.shape()[0], B.ptr(), B.shape()[0], A.shape()[1], factAB, factC, 0, 1) == 0);
}

template <>
inline void avg_diagonals(tensor<float, host_memory_space>& dst, const dia_matrix<float, host_memory_space>& dia) {
    cuvAssert(dia.num_dia() == (int)dst.size());
    cuvAssert(oracle_avg_diagonals(dst.ptr(), dia.vec().ptr(), dia.get_offsets().ptr(), dia.num_dia(), dia.h(), dia.w(),
                                   dia.stride(), dia.row_fact()) == 0);
}

namespace detail {
inline void reduce_host(void* v, int v_type, const void* m, int m_type, long long n_contig, long long n_strided,
                        bool over_strided, reduce_functor rf, float factNew, float factOld) {
    if (v_type == CUVDIA_T_F32 && m_type == CUVDIA_T_F32) {
        cuvAssert(oracle_reduce((float*)v, (const float*)m, n_contig, n_strided, over_strided ? 1 : 0, (int)rf, factNew,
                                factOld, 1) == 0);
    } else {
        cuvAssert(oracle_reduce_typed(v, v_type, m, m_type, n_contig, n_strided, over_strided ? 1 : 0, (int)rf, factNew,
                                      factOld) == 0);
    }
}
inline void learn_step_host(float* W, const float* dW, unsigned long long n, float learnrate, float decay) {
    oracle_learn_step_weight_decay(W, dW, (long)n, learnrate, decay);
}
inline void learn_step_momentum_host(float* W, float* momentum, const float* dW, unsigned long long n, float learnrate,
                                     float momentum_weight, float decay) {
    oracle_learn_step_weight_decay_momentum(W, momentum, dW, (long)n, learnrate, momentum_weight, decay, 1);
}
}  // namespace detail

}  // namespace cuv
