// densedense_to_dia and its block descriptors (matrix_ops/densedense_to_sparse.hpp:52-139 in CUV).
// CUV's device descriptor is a host-built list of the 16x16 tiles a diagonal crosses; the kernels
// behind this surface need no tile list, so the descriptor keeps its interface (constructor from a
// matrix, len(), blocks()) and carries nothing.
#pragma once
#include "cuv/basics/dia_matrix.hpp"
#include "cuv/basics/tensor.hpp"

#define SPARSE_DIA_BLOCK_SIZE 16
#define SPARSE_DIA_BLOCK_SIZE_LEN (2 * SPARSE_DIA_BLOCK_SIZE + 2)

namespace cuv {

template <class V, class I = unsigned int>
class host_block_descriptor {
  public:
    typedef dia_matrix<V, host_memory_space, I> diamat_type;
    host_block_descriptor(const diamat_type&) {}
};

template <class V, class I = unsigned int>
class dev_block_descriptor {
  public:
    typedef dia_matrix<V, dev_memory_space, I> diamat_type;
    struct block_array { int* ptr; int len; };
    explicit dev_block_descriptor(const diamat_type& d) { m_blocks.ptr = nullptr; m_blocks.len = 0; (void)d.plan(); }
    const block_array& blocks() const { return m_blocks; }
    int len() const { return m_blocks.len; }
  private:
    block_array m_blocks;
};

template <class V, class L, class I>
void densedense_to_dia(dia_matrix<V, dev_memory_space, I>& C, const dev_block_descriptor<V, I>&,
                       const tensor<V, dev_memory_space, L>& A, const tensor<V, dev_memory_space, L>& B,
                       const V& factAB = 1.f, const V& factC = 0.f) {
    static_assert(std::is_same<V, float>::value && std::is_same<L, column_major>::value,
                  "densedense_to_dia is implemented for float column-major operands");
    cuvAssert(A.shape().size() == 2);                    // matrix_ops/densedense_to_sparse.cu:261-262,276-278
    cuvAssert(B.shape().size() == 2);
    cuvAssert(C.w() == B.shape()[0]);
    cuvAssert(C.h() == A.shape()[0]);
    cuvAssert(A.shape()[1] == B.shape()[1]);
    cuvdia_check(cuvdia_dd2dia_f32(C.plan(), C.vec().ptr(), A.ptr(), (int)A.shape()[0], B.ptr(), (int)B.shape()[0],
                                   (int)A.shape()[1], factAB, factC, 0));
    cuvSafeCall(cudaDeviceSynchronize());
    cuvdia_check_plan(C.plan());
}

// host twin: CUV's own host code (the parity reference), not part of this library
template <class V, class L, class I>
void densedense_to_dia(dia_matrix<V, host_memory_space, I>& C, const host_block_descriptor<V, I>&,
                       const tensor<V, host_memory_space, L>& A, const tensor<V, host_memory_space, L>& B,
                       const V& factAB = 1.f, const V& factC = 0.f);

}  // namespace cuv
