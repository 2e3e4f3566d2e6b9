// avg_diagonals of the CUV surface (matrix_ops/diagonals.hpp:12 in CUV): dst[k] = mean of stored diagonal k.
// The device version calls the cuvdia C ABI, which follows the definition of CUV's host code (mean over the cells
// inside the matrix, matrix_ops/diagonals.cu:23-48); the host version is CUV's own code and is not part of this
// library (the test suite supplies it).
#pragma once
#include "cuv/basics/dia_matrix.hpp"
#include "cuv/basics/tensor.hpp"

namespace cuv {

template <class T, class M>
void avg_diagonals(tensor<T, M>& dst, const dia_matrix<T, M>& dia);

template <>
void avg_diagonals(tensor<float, host_memory_space>& dst, const dia_matrix<float, host_memory_space>& dia);

template <>
inline void avg_diagonals(tensor<float, dev_memory_space>& dst, const dia_matrix<float, dev_memory_space>& dia) {
    cuvAssert(dia.row_fact() == 1);                      // matrix_ops/diagonals.cu:28
    cuvAssert(dia.num_dia() == (int)dst.size());         // :29
    cuvdia_check(cuvdia_avg_diagonals_f32(dia.plan(), dia.vec().ptr(), dst.ptr(), 0));
    cuvSafeCall(cudaDeviceSynchronize());
}

}  // namespace cuv
