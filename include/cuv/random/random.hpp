// fill_rnd_uniform / rnd_binarize of the CUV surface (random/random.hpp:48-78 in CUV) for float device tensors.
// CUV draws with one generator state per thread, so its numbers depend on the launch geometry; here the number of an
// element is a pure function of (seed, draw count, element) - see cuvdia_uniform_f32 in cuvdia.h - which a host
// restatement reproduces.  initialize_mersenne_twister_seeds keeps its name: it sets the seed and starts the count of
// draws again.  A tensor is taken in memory order: the first dimension of a column-major tensor (the last of a
// row-major one) is the row of the generator's (row, column) pair.
#pragma once
#include <type_traits>

#include "cuv/basics/tensor.hpp"
#include "cuv/tools/cuv_general.hpp"

namespace cuv {

namespace detail {
struct rnd_state { unsigned long long seed = 0, draws = 0; };
inline rnd_state& rnd() { static rnd_state s; return s; }
template <class L> inline void rnd_shape(const tensor<float, dev_memory_space, L>& v, int* rows, int* cols) {
    const size_t nd = v.shape().size();
    const size_t fast = nd < 2 ? v.size() : std::is_same<L, column_major>::value ? v.shape()[0] : v.shape()[nd - 1];
    *rows = (int)fast;
    *cols = fast ? (int)(v.size() / fast) : 0;
}
}  // namespace detail

inline void initialize_mersenne_twister_seeds(unsigned int seed = 0) { detail::rnd().seed = seed; detail::rnd().draws = 0; }
inline void deinit_rng(unsigned int = 0) {}

// every element a uniform number in [0, 1); the next call draws other numbers
template <class L> void fill_rnd_uniform(tensor<float, dev_memory_space, L>& v) {
    int rows, cols;
    detail::rnd_shape(v, &rows, &cols);
    if (!rows) return;
    cuvdia_draw d = {detail::rnd().seed, detail::rnd().draws++, 0};
    cuvdia_check(cuvdia_uniform_f32(v.ptr(), rows, rows, cols, &d, 0, 0));
    cuvSafeCall(cudaDeviceSynchronize());
}

// every element x becomes 1 if x > u and 0 otherwise, u uniform in [0, 1)
template <class L> void rnd_binarize(tensor<float, dev_memory_space, L>& v) {
    int rows, cols;
    detail::rnd_shape(v, &rows, &cols);
    if (!rows) return;
    cuvdia_draw d = {detail::rnd().seed, detail::rnd().draws++, 0};
    cuvdia_check(cuvdia_rnd_binarize_f32(v.ptr(), rows, rows, cols, &d, 0, 0));
    cuvSafeCall(cudaDeviceSynchronize());
}

}  // namespace cuv
