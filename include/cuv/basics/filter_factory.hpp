// filter_factory of the CUV surface (basics/filter_factory.hpp:6-84 in CUV): builds the DIA matrix of a layer of
// fs x fs convolution filters between input_maps and output_maps images of px x py pixels - runs of fs consecutive
// diagonals, one image line (px) apart, one block of fs*fs diagonals per map distance - and reads one filter back out of
// such a matrix.  Host-side index arithmetic only; the matrices it makes are what the run-walking prod kernel and the
// run-aware densedense_to_dia kernel are built for.
#pragma once
#include <algorithm>
#include <vector>

#include "cuv/basics/dia_matrix.hpp"
#include "cuv/basics/tensor.hpp"

namespace cuv {

template <class T, class M, class I = unsigned int>
class filter_factory {
  public:
    typedef T value_type;
    typedef M memory_space;
    typedef I index_type;

    filter_factory(int px, int py, int fs, int input_maps, int output_maps)
        : m_px(px), m_py(py), m_fs(fs), m_input_maps(input_maps), m_output_maps(output_maps), m_dias_per_filter(fs * fs) {}

    // Diagonal numbers in storage order: for every map distance m = 0 .. output_maps + input_maps - 2 the fs*fs numbers
    // i*px + j (filter row i, filter column j) + m*px*py, all shifted so that the filter is centred on its pixel and the
    // first block belongs to the last input map (basics/filter_factory.hpp:58-71).
    std::vector<int> offsets() const {
        const int blocks = m_output_maps + m_input_maps - 1;
        const int shift = -(m_px + 1) * (m_fs / 2) - (m_input_maps - 1) * m_px * m_py;
        std::vector<int> off;
        off.reserve((size_t)blocks * m_fs * m_fs);
        for (int m = 0; m < blocks; m++)
            for (int i = 0; i < m_fs; i++)
                for (int j = 0; j < m_fs; j++) off.push_back(i * m_px + j + m * m_px * m_py + shift);
        return off;
    }

    // A new (px*py*input_maps) x (px*py*output_maps) matrix with those diagonals; the caller owns it.
    dia_matrix<T, M, I>* get_dia() {
        const std::vector<int> off = offsets();
        const int h = m_px * m_py * m_input_maps, w = m_px * m_py * m_output_maps;
        dia_matrix<T, M, I>* mat = new dia_matrix<T, M, I>(h, w, (int)off.size(), std::max(h, w));
        mat->set_offsets(off);
        return mat;
    }

    // The coefficients column `filternumber` of the matrix receives from each input map, in row order, as an
    // (fs*fs) x input_maps row-major tensor filled flat, map after map (basics/filter_factory.hpp:22-41); the caller owns it.
    template <class M2>
    tensor<T, M, row_major>* extract_filter(const dia_matrix<T, M2, I>& dia, unsigned int filternumber) {
        tensor<T, M, row_major>* mat = new tensor<T, M, row_major>(extents[m_fs * m_fs][m_input_maps]);
        for (unsigned int t = 0; t < mat->size(); t++) (*mat)[t] = (T)0;
        const unsigned int map_size = dia.h() / m_input_maps;
        for (unsigned int map = 0; map < (unsigned int)m_input_maps; map++) {
            unsigned int found = 0;
            for (unsigned int i = 0; i < map_size; i++) {
                const unsigned int row = i + map * map_size;
                if (!dia.has(row, filternumber)) continue;
                (*mat)[map * m_fs * m_fs + found++] = dia(row, filternumber);
                if (found >= mat->size()) break;
            }
        }
        return mat;
    }

  private:
    int m_px, m_py, m_fs, m_input_maps, m_output_maps;
    int m_dias_per_filter;
};

}  // namespace cuv
