// Dense tensor of the CUV surface: the subset of basics/tensor.hpp:188-1248 that the DIA path and
// its tests use.  Densely packed, 1-D or 2-D (n-D shapes are kept but only flat access is offered),
// shared ownership of the storage (same-type assignment aliases, tensor.hpp:881-890), copying
// assignment across memory spaces (:927-930), non-owning views on raw pointers (:834-854).
#pragma once
#include <cstring>
#include <memory>
#include <vector>

#include "cuv/basics/tags.hpp"
#include "cuv/tools/cuv_general.hpp"

namespace cuv {

// ---- shape helpers that stand in for the boost::multi_array generators CUV uses -------------------
struct index_range {
    long lo, hi;
    index_range(long a, long b) : lo(a), hi(b) {}
};
template <int N> struct index_gen {
    long lo[N > 0 ? N : 1], hi[N > 0 ? N : 1];
    index_gen<N + 1> operator[](const index_range& r) const {
        index_gen<N + 1> g;
        for (int i = 0; i < N; i++) { g.lo[i] = lo[i]; g.hi[i] = hi[i]; }
        g.lo[N] = r.lo; g.hi[N] = r.hi;
        return g;
    }
};
template <int N> struct extent_gen {
    unsigned ext[N > 0 ? N : 1];
    extent_gen<N + 1> operator[](unsigned e) const {
        extent_gen<N + 1> g;
        for (int i = 0; i < N; i++) g.ext[i] = ext[i];
        g.ext[N] = e;
        return g;
    }
};
static const index_gen<0> indices = index_gen<0>();
static const extent_gen<0> extents = extent_gen<0>();

// ---- raw storage ---------------------------------------------------------------------------------------
template <class V, class M> struct memory_ops;
template <class V> struct memory_ops<V, host_memory_space> {
    static V* alloc(size_t n) { return n ? static_cast<V*>(::operator new(n * sizeof(V))) : nullptr; }
    static void free(V* p) { ::operator delete(p); }
};
template <class V> struct memory_ops<V, dev_memory_space> {
    static V* alloc(size_t n) {
        void* p = nullptr;
        if (n) cuvSafeCall(cudaMalloc(&p, n * sizeof(V)));
        return static_cast<V*>(p);
    }
    static void free(V* p) { if (p) cudaFree(p); }
};
template <class M1, class M2> struct copy_kind;
template <> struct copy_kind<host_memory_space, host_memory_space> { static const cudaMemcpyKind value = cudaMemcpyHostToHost; };
template <> struct copy_kind<dev_memory_space, host_memory_space> { static const cudaMemcpyKind value = cudaMemcpyHostToDevice; };
template <> struct copy_kind<host_memory_space, dev_memory_space> { static const cudaMemcpyKind value = cudaMemcpyDeviceToHost; };
template <> struct copy_kind<dev_memory_space, dev_memory_space> { static const cudaMemcpyKind value = cudaMemcpyDeviceToDevice; };

template <class Mdst, class Msrc, class V>
inline void copy_raw(V* dst, const V* src, size_t n) {
    if (!n) return;
    if (copy_kind<Mdst, Msrc>::value == cudaMemcpyHostToHost) std::memcpy(dst, src, n * sizeof(V));
    else cuvSafeCall(cudaMemcpy(dst, src, n * sizeof(V), copy_kind<Mdst, Msrc>::value));
}

// Proxy for one element that may live on the device (basics/reference.hpp:52-201).
template <class V, class M> class reference {
    V* m_p;
  public:
    explicit reference(V* p) : m_p(p) {}
    operator V() const { V v; copy_raw<host_memory_space, M>(&v, m_p, 1); return v; }
    reference& operator=(const V& v) { copy_raw<M, host_memory_space>(m_p, &v, 1); return *this; }
    reference& operator=(const reference& o) { return *this = (V)o; }
    reference& operator+=(const V& v) { return *this = (V)(*this) + v; }
};

template <class V, class M, class L = row_major>
class tensor {
  public:
    typedef V value_type;
    typedef M memory_space_type;
    typedef L memory_layout_type;
    typedef unsigned int size_type;
    typedef int index_type;
    typedef reference<V, M> reference_type;

  private:
    std::vector<size_type> m_shape;
    std::shared_ptr<V> m_mem;     // null for views
    V* m_ptr;

    void allocate() {
        const size_t n = size();
        V* p = memory_ops<V, M>::alloc(n);
        m_mem = std::shared_ptr<V>(p, [](V* q) { memory_ops<V, M>::free(q); });
        m_ptr = p;
    }

  public:
    tensor() : m_ptr(nullptr) {}
    explicit tensor(size_type n) : m_shape(1, n), m_ptr(nullptr) { allocate(); }
    tensor(size_type h, size_type w) : m_ptr(nullptr) { m_shape.push_back(h); m_shape.push_back(w); allocate(); }
    template <int N> explicit tensor(const extent_gen<N>& e) : m_shape(e.ext, e.ext + N), m_ptr(nullptr) { allocate(); }
    explicit tensor(const std::vector<size_type>& shape) : m_shape(shape), m_ptr(nullptr) { allocate(); }
    // non-owning view on existing memory (tensor.hpp:834-854)
    template <int N> tensor(const index_gen<N>& idx, V* ptr) : m_ptr(ptr) {
        for (int i = 0; i < N; i++) m_shape.push_back((size_type)(idx.hi[i] - idx.lo[i]));
    }
    // copy construction / same-type assignment alias the storage
    tensor(const tensor&) = default;
    tensor& operator=(const tensor&) = default;
    // assignment from another memory space or layout copies (the element order in memory is kept)
    template <class M2, class L2> tensor(const tensor<V, M2, L2>& o) : m_ptr(nullptr) { *this = o; }
    template <class M2, class L2> tensor& operator=(const tensor<V, M2, L2>& o) {
        if (size() != o.size() || !m_ptr) { m_shape = o.shape(); allocate(); }
        else m_shape = o.shape();
        copy_raw<M, M2>(m_ptr, o.ptr(), o.size());
        return *this;
    }

    const std::vector<size_type>& shape() const { return m_shape; }
    size_type shape(size_t i) const { return m_shape[i]; }
    size_type ndim() const { return (size_type)m_shape.size(); }
    size_type size() const {
        if (m_shape.empty()) return 0;
        size_t n = 1;
        for (size_t i = 0; i < m_shape.size(); i++) n *= m_shape[i];
        return (size_type)n;
    }
    size_t memsize() const { return (size_t)size() * sizeof(V); }
    V* ptr() { return m_ptr; }
    const V* ptr() const { return m_ptr; }

    // flat access in memory order (tensor.hpp:439-472 reduces to this for densely packed tensors)
    reference_type operator[](index_type idx) { return reference_type(m_ptr + idx); }
    const reference_type operator[](index_type idx) const { return reference_type(m_ptr + idx); }
    reference_type operator()(index_type i) { return reference_type(m_ptr + i); }
    const reference_type operator()(index_type i) const { return reference_type(m_ptr + i); }
    reference_type operator()(index_type i, index_type j) { return reference_type(m_ptr + offset2(i, j)); }
    const reference_type operator()(index_type i, index_type j) const { return reference_type(m_ptr + offset2(i, j)); }
    reference_type operator()(index_type i, index_type j, index_type k) { return reference_type(m_ptr + offset3(i, j, k)); }
    const reference_type operator()(index_type i, index_type j, index_type k) const {
        return reference_type(m_ptr + offset3(i, j, k));
    }

  private:
    // element (i, j, k) of a 3-D tensor: the last index runs fastest in row-major storage, the first in column-major
    size_t offset3(index_type i, index_type j, index_type k) const {
        return std::is_same<L, column_major>::value ? ((size_t)k * m_shape[1] + j) * m_shape[0] + i
                                                    : ((size_t)i * m_shape[1] + j) * m_shape[2] + k;
    }
    size_t offset2(index_type i, index_type j) const {
        return std::is_same<L, column_major>::value ? (size_t)j * m_shape[0] + i : (size_t)i * m_shape[1] + j;
    }
};

}  // namespace cuv
