"""Rebuilds ``reference_fixtures.npz``: the known-answer cases CUV's own tests hold for the DIA path.

The reference's fixtures are parametric (sizes, offsets -3..3, ``sequence`` fill = 0,1,2,...), not
data files, and its tests pin the DIA routines by requiring "DIA result == dense result".  This
script rebuilds each fixture from its definition and computes the expected answer with a dense
float64 numpy computation that shares no code with the oracle or the CUDA kernels:

* ``spmv_*``   src/tests/spmv.cpp:49-52,65-97 (32x16, 7 diagonals, stride 32, rf 1, B 16x6, C 32x6)
               cases :103-115 (A^T*C, factors 1/0), :116-136 (A*B, 2/1.3), :137-143 (A^T*C, 2/1.3)
* ``dd2dia_*`` src/tests/densedense_to_dia.cpp:50-53,66-103,109-197 (36x19, rf 4, batch 16)
* ``diamat_*`` src/tests/dia_mat.cpp:48-79,111-119 (32x16, offsets 0,1,-1: dense(i,j) == dia(i,j))
* ``reduce_*`` src/tests/matrix_op.cpp:858-924 (270x270 uniform data, both axes, vs explicit sums)

Run:  python tests/golden/make_golden.py
"""
import os

import numpy as np


def dia_dense(h, w, rf, stride, offsets, vals):
    """dense(i,j) = vals[slot(j - i//rf)*stride + i], 0 where the diagonal is not stored
    (the definition of dia_matrix::operator(), basics/dia_matrix.hpp:236-243)."""
    slot = {int(k): s for s, k in enumerate(offsets)}
    d = np.zeros((h, w), dtype=np.float64)
    for i in range(h):
        for j in range(w):
            s = slot.get(j - i // rf)
            if s is not None:
                d[i, j] = vals[s * stride + i]
    return d


def seq(*shape):
    """``sequence`` on a column-major tensor: element with linear memory index n holds n."""
    n = int(np.prod(shape))
    return np.arange(n, dtype=np.float64).reshape(shape, order="F")


def main():
    out = {}
    # ---- spmv.cpp ----
    n, m, k, rf = 32, 16, 6, 1
    offs = np.arange(-3, 4, dtype=np.int32)
    stride = max(n, m)
    avals = np.arange(7 * stride, dtype=np.float64)
    A = dia_dense(n, m, rf, stride, offs, avals)
    B, C = seq(m, k), seq(n, k)
    out.update(spmv_h=n, spmv_w=m, spmv_rf=rf, spmv_stride=stride, spmv_offsets=offs,
               spmv_vals=avals.astype(np.float32), spmv_B=B.astype(np.float32), spmv_C=C.astype(np.float32),
               spmv_dense=A.astype(np.float32),
               spmv_expect_t_1_0=A.T @ C,                     # prod(B, A, C, 't') defaults
               spmv_expect_n_2_13=np.float32(1.3) * C + 2.0 * (A @ B),   # prod(C, A, B, 'n', 2, 1.3)
               spmv_expect_t_2_13=np.float32(1.3) * B + 2.0 * (A.T @ C))  # prod(B, A, C, 't', 2, 1.3)
    # ---- densedense_to_dia.cpp ----
    n, m, k, rf = 36, 19, 16, 4
    stride = max(n, m)
    X, H = seq(n, k), seq(m, k)
    dense = X @ H.T
    expect = np.zeros(7 * stride, dtype=np.float64)
    mask = np.zeros(7 * stride, dtype=bool)
    slot = {int(kk): s for s, kk in enumerate(offs)}
    for i in range(n):
        for j in range(m):
            s = slot.get(j - i // rf)
            if s is not None:
                expect[s * stride + i] = dense[i, j]
                mask[s * stride + i] = True
    out.update(dd2dia_h=n, dd2dia_w=m, dd2dia_rf=rf, dd2dia_stride=stride, dd2dia_offsets=offs,
               dd2dia_A=X.astype(np.float32), dd2dia_B=H.astype(np.float32),
               dd2dia_expect=expect, dd2dia_mask=mask)
    # ---- dia_mat.cpp ----
    n, m = 32, 16
    offs3 = np.array([0, 1, -1], dtype=np.int32)
    v3 = np.arange(3 * 32, dtype=np.float64)
    out.update(diamat_h=n, diamat_w=m, diamat_stride=32, diamat_offsets=offs3, diamat_vals=v3.astype(np.float32),
               diamat_dense=dia_dense(n, m, 1, 32, offs3, v3).astype(np.float32))
    # ---- matrix_op.cpp all_reduce ----
    rng = np.random.Generator(np.random.PCG64(270))
    M = np.asfortranarray(rng.random((270, 270), dtype=np.float32))
    M64 = M.astype(np.float64)
    out.update(reduce_src=M,
               reduce_add_over_cols=M64.sum(axis=1), reduce_add_over_rows=M64.sum(axis=0),
               reduce_max_over_cols=M64.max(axis=1), reduce_max_over_rows=M64.max(axis=0),
               reduce_min_over_cols=M64.min(axis=1), reduce_min_over_rows=M64.min(axis=0),
               reduce_argmax_over_cols=M64.argmax(axis=1), reduce_argmax_over_rows=M64.argmax(axis=0),
               reduce_argmin_over_cols=M64.argmin(axis=1), reduce_argmin_over_rows=M64.argmin(axis=0),
               reduce_logaddexp_over_cols=np.log(np.exp(M64).sum(axis=1)),
               reduce_logaddexp_over_rows=np.log(np.exp(M64).sum(axis=0)),
               reduce_addsq_over_cols=(M64 ** 2).sum(axis=1), reduce_addsq_over_rows=(M64 ** 2).sum(axis=0))
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_fixtures.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
