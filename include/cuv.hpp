// Umbrella header of the CUV surface for the DIA sparse path.
#pragma once
#include "cuv/basics/dia_matrix.hpp"
#include "cuv/basics/filter_factory.hpp"
#include "cuv/basics/sparse_matrix_io.hpp"
#include "cuv/basics/tags.hpp"
#include "cuv/basics/tensor.hpp"
#include "cuv/convert/convert.hpp"
#include "cuv/matrix_ops/densedense_to_sparse.hpp"
#include "cuv/matrix_ops/diagonals.hpp"
#include "cuv/matrix_ops/matrix_ops.hpp"
#include "cuv/tensor_ops/rprop.hpp"
#include "cuv/tensor_ops/tensor_ops.hpp"
#include "cuv/tools/cuv_general.hpp"
