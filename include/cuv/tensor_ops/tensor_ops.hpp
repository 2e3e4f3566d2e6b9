// fill / sequence / apply_binary_functor of the CUV surface (tensor_ops/tensor_ops.hpp:108-122,
// 460-492, 530-655 in CUV) for float tensors: the functors the DIA path's callers use (ADD,
// SUBTRACT, MULT, AXPY, XPBY, AXPBY).  Device tensors go through the cuvdia C ABI; host tensors are
// plain loops (data set-up, not part of the accelerated path).
#pragma once
#include "cuv/basics/tensor.hpp"

namespace cuv {

enum BinaryFunctor { BF_ADD = CUVDIA_BF_ADD, BF_SUBTRACT = CUVDIA_BF_SUBTRACT, BF_MULT = CUVDIA_BF_MULT,
                     BF_AXPY = CUVDIA_BF_AXPY, BF_XPBY = CUVDIA_BF_XPBY, BF_AXPBY = CUVDIA_BF_AXPBY };

namespace detail {
inline float apply_bf(BinaryFunctor bf, float a, float b, float p, float p2) {
    switch (bf) {
        case BF_ADD: return a + b;
        case BF_SUBTRACT: return a - b;
        case BF_MULT: return a * b;
        case BF_AXPY: return p * a + b;       // functors.hpp:412-418
        case BF_XPBY: return a + p * b;       // functors.hpp:419-425
        default: return p * a + p2 * b;       // functors.hpp:426-433
    }
}
template <class L>
void binary(tensor<float, host_memory_space, L>& dst, const tensor<float, host_memory_space, L>& x,
            const tensor<float, host_memory_space, L>& y, BinaryFunctor bf, float p, float p2) {
    cuvAssert(dst.size() == x.size() && x.size() == y.size());
    float* d = dst.ptr(); const float* a = x.ptr(); const float* b = y.ptr();
    for (unsigned i = 0; i < dst.size(); i++) d[i] = apply_bf(bf, a[i], b[i], p, p2);
}
template <class L>
void binary(tensor<float, dev_memory_space, L>& dst, const tensor<float, dev_memory_space, L>& x,
            const tensor<float, dev_memory_space, L>& y, BinaryFunctor bf, float p, float p2) {
    cuvAssert(dst.size() == x.size() && x.size() == y.size());
    cuvdia_check(cuvdia_binary_f32(dst.ptr(), x.ptr(), y.ptr(), (int)bf, p, p2, dst.size(), 0));
    cuvSafeCall(cudaDeviceSynchronize());
}
}  // namespace detail

// dst = bf(dst, src)
template <class M, class L>
void apply_binary_functor(tensor<float, M, L>& dst, const tensor<float, M, L>& src, BinaryFunctor bf, float p = 0.f,
                          float p2 = 0.f) { detail::binary(dst, dst, src, bf, p, p2); }
// dst = bf(src1, src2)
template <class M, class L>
void apply_binary_functor(tensor<float, M, L>& dst, const tensor<float, M, L>& src1, const tensor<float, M, L>& src2,
                          BinaryFunctor bf, float p = 0.f, float p2 = 0.f) { detail::binary(dst, src1, src2, bf, p, p2); }

template <class V, class L, class S> void fill(tensor<V, host_memory_space, L>& v, const S& p) {
    V* d = v.ptr();
    for (unsigned i = 0; i < v.size(); i++) d[i] = (V)p;
}
template <class L, class S> void fill(tensor<float, dev_memory_space, L>& v, const S& p) {
    cuvdia_check(cuvdia_fill_f32(v.ptr(), (float)p, v.size(), 0));
    cuvSafeCall(cudaDeviceSynchronize());
}
// 0, 1, 2, ... in memory order (thrust::sequence in CUV, tensor_ops.cuh:251-252)
template <class V, class L> void sequence(tensor<V, host_memory_space, L>& v) {
    V* d = v.ptr();
    for (unsigned i = 0; i < v.size(); i++) d[i] = (V)i;
}
template <class L> void sequence(tensor<float, dev_memory_space, L>& v) {
    cuvdia_check(cuvdia_sequence_f32(v.ptr(), v.size(), 0));
    cuvSafeCall(cudaDeviceSynchronize());
}

}  // namespace cuv
