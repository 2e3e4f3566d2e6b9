// dia_matrix of the CUV surface (basics/dia_matrix.hpp:57-276 in CUV): num_dia diagonals of `stride`
// values stored back to back in one 1-D tensor, int offsets in the caller's order, a host-side map
// diagonal -> slot, and the row factor ("steepness").  Cell (i,j) is vec[slot(j - i/rf)*stride + i].
// The device specialisation additionally carries the cuvdia plan the kernels need (created on
// demand, dropped when the offsets change).
#pragma once
#include <algorithm>
#include <map>
#include <vector>

#include "cuv/basics/tensor.hpp"

namespace cuv {

template <class V, class M, class I = unsigned int>
class dia_matrix {
  public:
    typedef V value_type;
    typedef M memory_space_type;
    typedef I index_type;
    typedef tensor<V, M> vec_type;
    typedef tensor<int, M> intvec_type;

  private:
    index_type m_height, m_width;
    int m_num_dia;
    unsigned int m_stride;
    vec_type* m_vec;
    intvec_type m_offsets;
    std::map<int, index_type> m_dia2off;
    int m_row_fact;
    mutable cuvdia_plan* m_plan;

    void drop_plan() const { if (m_plan) { cuvdia_plan_destroy(m_plan); m_plan = nullptr; } }

  public:
    dia_matrix() : m_height(0), m_width(0), m_num_dia(0), m_stride(0), m_vec(nullptr), m_row_fact(0), m_plan(nullptr) {}
    dia_matrix(const index_type& h, const index_type& w, const int& num_dia, const int& stride, int row_fact = 1)
        : m_height(h), m_width(w), m_num_dia(num_dia), m_stride(stride), m_vec(nullptr), m_offsets(num_dia),
          m_row_fact(row_fact), m_plan(nullptr) {
        cuvAssert(m_row_fact > 0);
        alloc();
    }
    ~dia_matrix() { dealloc(); drop_plan(); }
    dia_matrix(const dia_matrix&) = delete;

    void alloc() {
        cuvAssert(m_stride >= m_height || m_stride >= m_width);
        m_vec = new vec_type(m_stride * m_num_dia);
    }
    void dealloc() { delete m_vec; m_vec = nullptr; }

    index_type h() const { return m_height; }
    index_type w() const { return m_width; }
    index_type n() const { return m_height * m_width; }
    std::vector<index_type> shape() const { return std::vector<index_type>{m_height, m_width}; }
    const vec_type& vec() const { return *m_vec; }
    vec_type& vec() { return *m_vec; }
    const vec_type* vec_ptr() const { return m_vec; }
    vec_type* vec_ptr() { return m_vec; }
    V* ptr() const { return m_vec->ptr(); }
    int num_dia() const { return m_num_dia; }
    unsigned int stride() const { return m_stride; }
    int row_fact() const { return m_row_fact; }

    template <class T> void set_offsets(T begin, const T& end) {
        int i = 0;
        while (begin != end) m_offsets[i++] = (int)*begin++;
        post_update_offsets();
    }
    template <class T> void set_offsets(const std::vector<T>& v) {
        for (unsigned int i = 0; i < v.size(); i++) m_offsets[i] = (int)v[i];
        post_update_offsets();
    }
    void post_update_offsets() {
        m_dia2off.clear();
        for (unsigned int i = 0; i < m_offsets.size(); ++i) m_dia2off[m_offsets[i]] = i;
        drop_plan();
    }
    void set_offset(const index_type& idx, const index_type& val) {
        m_offsets[idx] = (int)val;
        m_dia2off[(int)val] = idx;
        drop_plan();
    }
    vec_type* get_dia(const int& k) {
        return new vec_type(indices[index_range(0, m_stride)], m_vec->ptr() + m_dia2off[k] * m_stride);
    }
    const intvec_type& get_offsets() const { return m_offsets; }
    intvec_type& get_offsets() { return m_offsets; }
    int get_offset(const index_type& idx) const { return m_offsets[idx]; }
    const std::map<int, index_type>& dia2off() const { return m_dia2off; }

    void set(const index_type& i, const index_type& j, const value_type& val) {
        auto it = m_dia2off.find((int)j - (int)i / m_row_fact);
        if (it == m_dia2off.end()) return;
        (*m_vec)[it->second * m_stride + i] = val;
    }
    value_type operator()(const index_type& i, const index_type& j) const {
        auto it = m_dia2off.find((int)j - (int)i / m_row_fact);
        if (it == m_dia2off.end()) return (value_type)0;
        return (*m_vec)[it->second * m_stride + i];
    }
    bool has(const index_type& i, const index_type& j) const {
        return m_dia2off.find((int)j - (int)i / m_row_fact) != m_dia2off.end();
    }

    // Assignment moves the storage out of the source, as in CUV (dia_matrix.hpp:259-275).
    dia_matrix& operator=(const dia_matrix& o) {
        if (this == &o) return *this;
        dealloc();
        drop_plan();
        m_height = o.m_height; m_width = o.m_width;
        m_vec = o.m_vec;
        m_num_dia = o.m_num_dia; m_stride = o.m_stride; m_row_fact = o.m_row_fact;
        m_offsets = o.m_offsets; m_dia2off = o.m_dia2off;
        const_cast<dia_matrix&>(o).m_vec = nullptr;
        return *this;
    }

    // The structure handle the device kernels take; only meaningful for dev_memory_space.
    cuvdia_plan* plan() const {
        if (!m_plan) {
            std::vector<int> off(m_num_dia);
            for (int i = 0; i < m_num_dia; ++i) off[i] = m_offsets[i];
            cuvdia_check(cuvdia_plan_create(&m_plan, (int)m_height, (int)m_width, m_num_dia, (int)m_stride, m_row_fact,
                                            off.data()));
        }
        return m_plan;
    }
};

}  // namespace cuv
