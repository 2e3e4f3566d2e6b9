// convert(dst, src) of the CUV surface (convert/convert.hpp:58-59, convert/convert.cu:42-112 in CUV):
// dense tensors between memory spaces, DIA matrices between memory spaces (offsets, values and the
// diagonal map), and a host DIA matrix to a host dense matrix.
#pragma once
#include <algorithm>

#include "cuv/basics/dia_matrix.hpp"
#include "cuv/basics/tensor.hpp"
#include "cuv/tensor_ops/tensor_ops.hpp"

namespace cuv {

template <class V, class M1, class M2, class L>
void convert(tensor<V, M1, L>& dst, const tensor<V, M2, L>& src) { dst = src; }

// host dia -> host dense (convert.cu:42-66)
template <class V, class L, class I>
void convert(tensor<V, host_memory_space, L>& dst, const dia_matrix<V, host_memory_space, I>& src) {
    if (dst.ndim() != 2 || dst.shape()[0] != src.h() || dst.shape()[1] != src.w())
        dst = tensor<V, host_memory_space, L>(src.h(), src.w());
    fill(dst, 0);
    const int rf = src.row_fact();
    for (int oi = 0; oi < src.num_dia(); oi++) {
        const int o = src.get_offset(oi);
        I j = (I)std::max(0, o), i = (I)(rf * std::max(0, -o));
        for (; i < src.h() && j < src.w(); j++)
            for (int k = 0; k < rf && i < src.h(); k++, i++) dst(i, j) = src(i, j);
    }
}

namespace detail {
template <class V, class M1, class M2, class I>
void convert_dia(dia_matrix<V, M1, I>& dst, const dia_matrix<V, M2, I>& src) {
    if (dst.h() != src.h() || dst.w() != src.w() || dst.row_fact() != src.row_fact() || !dst.vec_ptr() ||
        dst.num_dia() != src.num_dia() || dst.stride() != src.stride())
        dst = dia_matrix<V, M1, I>(src.h(), src.w(), src.num_dia(), src.stride(), src.row_fact());
    cuvAssert(dst.vec_ptr());
    cuvAssert(src.vec_ptr());
    dst.get_offsets() = src.get_offsets();       // copies across memory spaces
    dst.vec() = src.vec();
    dst.post_update_offsets();
}
}  // namespace detail

// host dia -> dev dia (convert.cu:71-90) and dev dia -> host dia (:95-112)
template <class V, class I>
void convert(dia_matrix<V, dev_memory_space, I>& dst, const dia_matrix<V, host_memory_space, I>& src) { detail::convert_dia(dst, src); }
template <class V, class I>
void convert(dia_matrix<V, host_memory_space, I>& dst, const dia_matrix<V, dev_memory_space, I>& src) { detail::convert_dia(dst, src); }

}  // namespace cuv
