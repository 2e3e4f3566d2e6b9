"""Saving and loading a DIA matrix: the seven fields CUV serialises (basics/sparse_matrix_io.hpp:59-72)
survive a round trip through the plain little-endian record (CUV's test: src/tests/dia_mat.cpp:84-101)."""
import numpy as np
import pytest


def test_host_round_trip(tmp_path):
    import cuv_b200 as cb
    rng = np.random.default_rng(3)
    m = cb.host_dia_matrix_f(32, 16, [0, 1, -1], 32, 1)
    m.vec[:] = rng.standard_normal(m.vec.size).astype(np.float32)
    fn = str(tmp_path / "w.dia")
    cb.save_dia_mat(m, fn)
    m2 = cb.load_dia_mat(fn)
    assert (m2.h, m2.w, m2.num_dia, m2.stride, m2.row_fact) == (32, 16, 3, 32, 1)
    assert np.array_equal(m2.offsets, m.offsets) and np.array_equal(m2.vec, m.vec)
    assert m2(5, 6) == m(5, 6) and m2(5, 9) == 0.0
    with open(fn, "r+b") as f:
        f.write(b"XXXX")
    with pytest.raises(cb.CuvDiaError):
        cb.load_dia_mat(fn)


@pytest.mark.gpu
def test_device_round_trip(tmp_path):
    import cuv_b200 as cb
    d = cb.dev_dia_matrix_f(64, 48, [3, -2, 0, 7], 64, 2)
    d.vec.normal_()
    fn = str(tmp_path / "d.dia")
    cb.save_dia_mat(d, fn)
    d2 = cb.load_dia_mat(fn, device="cuda")
    assert (d2.h, d2.w, d2.row_fact, d2.stride) == (64, 48, 2, 64)
    assert np.array_equal(d2.offsets, d.offsets)
    assert np.array_equal(d2.vec.cpu().numpy(), d.vec.cpu().numpy())


def test_filter_factory_offsets_and_extraction():
    """filter_factory (basics/filter_factory.hpp:43-76): the diagonal numbers of a convolution layer - for the
    reference's speed fixture (src/tests/spmv_speed.cpp:96-104 stores i*px + j once per map) the un-shifted pattern -
    and a filter written into the matrix comes back out of it."""
    import cuv_b200 as cb
    ff = cb.filter_factory(16, 16, 5, 2, 3)
    offs = ff.offsets()
    want = np.array([i * 16 + j + m * 256 for m in range(4) for i in range(5) for j in range(5)], dtype=np.int32)
    assert np.array_equal(offs, want - 17 * 2 - 256)
    mat = ff.get_dia(device=None)
    assert (mat.h, mat.w, mat.num_dia, mat.stride) == (512, 768, 100, 768)
    # one map in, one map out: column 100 of the matrix holds the 3 x 3 filter centred on pixel 100
    ff1 = cb.filter_factory(12, 12, 3, 1, 1)
    m1 = ff1.get_dia(device=None)
    m1.vec[:] = 0
    filt = np.arange(1, 10, dtype=np.float32)
    col = 100
    for t, off in enumerate(ff1.offsets().tolist()):
        m1.set(col - off, col, filt[t])          # cell (i, i + off) lies in column `col` for i = col - off
    got = ff1.extract_filter(m1, col)
    # rows ascend while the diagonals that hit the column descend: the filter comes back reversed
    assert got.shape == (9, 1) and np.array_equal(got[:, 0], filt[::-1])
