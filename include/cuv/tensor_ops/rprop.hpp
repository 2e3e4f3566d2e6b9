// learn_step_weight_decay / learn_step_weight_decay_momentum of the CUV surface
// (tensor_ops/rprop.hpp:117-155 in CUV) for float tensors and, as the sparse RBM's update step uses
// them (examples/rbm/base.py:72-75), for DIA matrices through their value vector.  Device tensors go
// through the cuvdia C ABI; the host_memory_space versions are declared only.
#pragma once
#include "cuv/basics/dia_matrix.hpp"
#include "cuv/basics/tensor.hpp"

namespace cuv {

namespace detail {
// host halves: not part of the accelerated path, supplied by whoever links a host implementation
void learn_step_host(float* W, const float* dW, unsigned long long n, float learnrate, float decay);
void learn_step_momentum_host(float* W, float* momentum, const float* dW, unsigned long long n, float learnrate,
                              float momentum_weight, float decay);
}  // namespace detail

// W = -learnrate*dW + (1 - learnrate*decay)*W.  sparsedecay has no effect, as in CUV (rprop.cu:147-156).
template <class L>
void learn_step_weight_decay(tensor<float, dev_memory_space, L>& W, const tensor<float, dev_memory_space, L>& dW,
                             const float& learnrate, const float& decay = 0.0f, const float& sparsedecay = 0.0f) {
    (void)sparsedecay;
    cuvAssert(dW.ptr());                                  // rprop.cu:342-344
    cuvAssert(W.ptr());
    cuvAssert(W.size() == dW.size());
    cuvdia_check(cuvdia_learn_step_weight_decay_f32(W.ptr(), dW.ptr(), W.size(), learnrate, decay, 0));
    cuvSafeCall(cudaDeviceSynchronize());
}
template <class L>
void learn_step_weight_decay(tensor<float, host_memory_space, L>& W, const tensor<float, host_memory_space, L>& dW,
                             const float& learnrate, const float& decay = 0.0f, const float& sparsedecay = 0.0f) {
    (void)sparsedecay;
    cuvAssert(dW.ptr());
    cuvAssert(W.ptr());
    cuvAssert(W.size() == dW.size());
    detail::learn_step_host(W.ptr(), dW.ptr(), W.size(), learnrate, decay);
}

// m = momentum_weight*m - learnrate*(dW + decay*W); W += m; momentum = m  (rprop.cu:158-170)
template <class L>
void learn_step_weight_decay_momentum(tensor<float, dev_memory_space, L>& W, tensor<float, dev_memory_space, L>& momentum,
                                      const tensor<float, dev_memory_space, L>& dW, const float& learnrate,
                                      const float& momentum_weight = 0.9f, const float& decay = 0.0f,
                                      const float& sparsedecay = 0.0f) {
    (void)sparsedecay;
    cuvAssert(dW.ptr());                                  // rprop.cu:371-374
    cuvAssert(W.ptr());
    cuvAssert(W.size() == dW.size());
    cuvAssert(W.size() == momentum.size());
    cuvdia_check(cuvdia_learn_step_weight_decay_momentum_f32(W.ptr(), momentum.ptr(), dW.ptr(), W.size(), learnrate,
                                                             momentum_weight, decay, 0));
    cuvSafeCall(cudaDeviceSynchronize());
}
template <class L>
void learn_step_weight_decay_momentum(tensor<float, host_memory_space, L>& W, tensor<float, host_memory_space, L>& momentum,
                                      const tensor<float, host_memory_space, L>& dW, const float& learnrate,
                                      const float& momentum_weight = 0.9f, const float& decay = 0.0f,
                                      const float& sparsedecay = 0.0f) {
    (void)sparsedecay;
    cuvAssert(W.size() == dW.size());
    cuvAssert(W.size() == momentum.size());
    detail::learn_step_momentum_host(W.ptr(), momentum.ptr(), dW.ptr(), W.size(), learnrate, momentum_weight, decay);
}

// The sparse weight matrix and its gradient share offsets and stride; the step runs over the whole
// value vector, padding cells included (they are never read by prod).
template <class M>
void learn_step_weight_decay(dia_matrix<float, M>& W, const dia_matrix<float, M>& dW, const float& learnrate,
                             const float& decay = 0.0f, const float& sparsedecay = 0.0f) {
    cuvAssert(W.num_dia() == dW.num_dia() && W.stride() == dW.stride());
    learn_step_weight_decay(W.vec(), dW.vec(), learnrate, decay, sparsedecay);
}

}  // namespace cuv
