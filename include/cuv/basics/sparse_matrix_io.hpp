// Saving and loading a host dia_matrix.  CUV serialises seven fields through Boost.Serialization -
// width, height, num_dia, stride, row_fact, offsets, values (basics/sparse_matrix_io.hpp:59-72); this
// surface writes the same fields in the same order as a plain little-endian record: an 8-byte tag
// "CUVDIA1\0", five int32, num_dia int32 offsets, num_dia*stride float32 values.
#pragma once
#include <cstdint>
#include <cstring>
#include <fstream>
#include <string>
#include <vector>

#include "cuv/basics/dia_matrix.hpp"

namespace cuv {

template <class I>
void save_dia_matrix(const dia_matrix<float, host_memory_space, I>& m, const std::string& filename) {
    std::ofstream f(filename.c_str(), std::ios::binary);
    cuvAssert(f.good());
    const char tag[8] = {'C', 'U', 'V', 'D', 'I', 'A', '1', '\0'};
    f.write(tag, 8);
    const int32_t head[5] = {(int32_t)m.w(), (int32_t)m.h(), (int32_t)m.num_dia(), (int32_t)m.stride(), (int32_t)m.row_fact()};
    f.write(reinterpret_cast<const char*>(head), sizeof(head));
    f.write(reinterpret_cast<const char*>(m.get_offsets().ptr()), sizeof(int32_t) * m.num_dia());
    f.write(reinterpret_cast<const char*>(m.vec().ptr()), sizeof(float) * (size_t)m.num_dia() * m.stride());
    cuvAssert(f.good());
}

template <class I>
void load_dia_matrix(dia_matrix<float, host_memory_space, I>& m, const std::string& filename) {
    std::ifstream f(filename.c_str(), std::ios::binary);
    cuvAssert(f.good());
    char tag[8];
    f.read(tag, 8);
    cuvAssert(std::memcmp(tag, "CUVDIA1", 8) == 0);
    int32_t head[5];
    f.read(reinterpret_cast<char*>(head), sizeof(head));
    cuvAssert(f.good());
    m = dia_matrix<float, host_memory_space, I>(head[1], head[0], head[2], head[3], head[4]);
    std::vector<int32_t> off(head[2]);
    f.read(reinterpret_cast<char*>(off.data()), sizeof(int32_t) * off.size());
    m.set_offsets(off);
    f.read(reinterpret_cast<char*>(m.vec().ptr()), sizeof(float) * (size_t)head[2] * head[3]);
    cuvAssert(f.good());
}

}  // namespace cuv
