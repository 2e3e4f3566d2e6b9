"""GPU parity: every C-ABI routine against the CPU oracle on identical seeded inputs.

prod in EXACT mode must be bit-identical to the oracle; prod in FAST mode within 1e-5 of the sum of
|terms| (fused multiply-add rounds once per term); densedense_to_dia and additive reductions within
1e-4*sqrt(batch/128) relative; index-valued and min/max reductions exactly."""
import numpy as np
import pytest

from oracle import host_oracle as ho
from tests.helpers import F, assert_bits_equal, make_dia, scattered_offsets, to_dev_dia

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def cb():
    import torch
    assert torch.cuda.is_available()
    import cuv_b200
    return cuv_b200


def run_prod(cb, A, B, C0, trans, fab, fc, mode):
    D = to_dev_dia(A)
    Bd, Cd = cb.to_device(B), cb.to_device(C0)
    before = cb.launch_count()
    cb.prod(Cd, D, Bd, trans, "n", fab, fc, mode)
    assert cb.launch_count() > before
    return cb.to_host(Cd)


def prod_case(cb, rng, h, w, offsets, rf, ncols, trans, fab, fc, stride=None):
    A = make_dia(rng, h, w, offsets, rf, stride)
    rb, rc = (h, w) if trans == "t" else (w, h)
    B = F(rng.uniform(-1, 1, (rb, ncols)))
    C0 = F(rng.uniform(-1, 1, (rc, ncols)))
    if fc == 0:
        C0[:] = np.nan                                   # factC == 0: C must never be read
    want = C0.copy(order="F")
    ho.prod(want, A, B, trans, fab, fc, nthreads=4)
    got = run_prod(cb, A, B, C0, trans, fab, fc, cb.MODE_EXACT)
    assert_bits_equal(got, want, "exact prod %s h=%d w=%d rf=%d nd=%d" % (trans, h, w, rf, len(offsets)))
    fast = run_prod(cb, A, B, C0, trans, fab, fc, cb.MODE_FAST)
    # bound: one rounding difference per term
    Aabs = ho.DiaHost(h, w, A.offsets, A.stride, rf, np.abs(np.nan_to_num(A.vals)))
    mag = F(np.abs(np.nan_to_num(C0)) * abs(fc))
    ho.prod(mag, Aabs, F(np.abs(B)), trans, abs(fab), 1.0, nthreads=4)
    assert np.all(np.abs(fast.astype(np.float64) - want) <= 1e-5 * mag + 1e-30)
    return got


def test_reference_fixture_spmv(cb, golden):
    g = golden                                           # src/tests/spmv.cpp:103-129
    A = ho.DiaHost(int(g["spmv_h"]), int(g["spmv_w"]), g["spmv_offsets"], int(g["spmv_stride"]), 1, g["spmv_vals"])
    B, C = F(g["spmv_B"]), F(g["spmv_C"])
    got = run_prod(cb, A, C, F(np.full_like(B, np.nan)), "t", 1.0, 0.0, cb.MODE_EXACT)
    assert np.array_equal(got.astype(np.float64), g["spmv_expect_t_1_0"])
    got = run_prod(cb, A, B, C, "n", 2.0, 1.3, cb.MODE_EXACT)
    np.testing.assert_allclose(got, g["spmv_expect_n_2_13"], rtol=1e-6)
    want = C.copy(order="F"); ho.prod(want, A, B, "n", 2.0, 1.3)
    assert_bits_equal(got, want)


@pytest.mark.parametrize("trans", ["n", "t"])
@pytest.mark.parametrize("rf", [1, 2, 4])
def test_prod_scattered_small(cb, trans, rf):
    rng = np.random.default_rng(100 + rf + 10 * (trans == "t"))
    w = 150
    h = 57 * rf
    offs = scattered_offsets(rng, 9, -(h // rf) + 1, w - 1, sort=False)   # user order, includes extreme diagonals
    prod_case(cb, rng, h, w, offs, rf, 13, trans, 1.5, 0.5, stride=h + 5)
    prod_case(cb, rng, h, w, offs, rf, 1, trans, 1.0, 0.0)


@pytest.mark.parametrize("trans", ["n", "t"])
@pytest.mark.parametrize("rf", [1, 2, 4])
@pytest.mark.parametrize("lo,nd", [(-8, 16), (-5, 11), (3, 40), (-70, 33)])
def test_prod_band_small(cb, trans, rf, lo, nd):
    rng = np.random.default_rng(7 * nd + rf + 1000 * (trans == "t"))
    w = 200
    h = 64 * rf
    offs = np.arange(lo, lo + nd, dtype=np.int32)
    prod_case(cb, rng, h, w, offs, rf, 24, trans, 1.0, 0.0)
    prod_case(cb, rng, h, w, offs, rf, 37, trans, 0.75, 2.0, stride=h + 12)


@pytest.mark.parametrize("trans", ["n", "t"])
def test_prod_band_ragged_sizes(cb, trans):
    rng = np.random.default_rng(31 + (trans == "t"))
    for h, w, ncols in [(257, 301, 65), (130, 97, 3), (1000, 1000, 129)]:
        offs = np.arange(-17, 23, dtype=np.int32)
        prod_case(cb, rng, h, w, offs, 1, ncols, trans, 1.0, 0.5)


@pytest.mark.parametrize("trans", ["n", "t"])
@pytest.mark.parametrize("h,w,lo,nd,ncols,fab,fc", [
    (1000, 1000, -64, 128, 1024, 1.0, 0.0),      # square, centred band, one full column tile
    (257, 301, -40, 97, 800, 0.75, 2.0),         # ragged rows, partly filled column tile, both factors
    (301, 257, 3, 130, 1000, 1.0, 0.5),          # band above the main diagonal (alignment shift 3)
    (640, 2000, 900, 200, 1024, 2.0, 0.0),       # wide matrix, band far from the main diagonal
    (2000, 640, -1500, 256, 2048, 1.0, 0.0),     # tall matrix, two column tiles
    (96, 96, -95, 191, 768, 1.0, 0.0),           # every diagonal of a small matrix: most cells outside it
])
def test_prod_band_wide_batches(cb, trans, h, w, lo, nd, ncols, fab, fc):
    """Bands times many batch columns (the streaming banded kernel: 32-row tiles, 1024 columns per block)."""
    rng = np.random.default_rng(h + 7 * nd + ncols + (trans == "t"))
    offs = np.arange(lo, lo + nd, dtype=np.int32)
    prod_case(cb, rng, h, w, offs, 1, ncols, trans, fab, fc)


@pytest.mark.parametrize("trans", ["n", "t"])
@pytest.mark.parametrize("h,w,rf,lo,nd,ncols,fab,fc", [
    (1024, 256, 4, -64, 128, 512, 1.0, 0.5),     # config 1's pattern at a quarter of the size
    (1024, 512, 2, -50, 100, 1024, 1.0, 0.0),    # row factor 2, one full column tile
    (2048, 256, 8, -30, 64, 300, 0.75, 2.0),     # row factor 8, a partly filled tile, both factors
    (1023, 256, 4, -7, 40, 256, 1.0, 0.0),       # height not a multiple of the row factor: the last group is cut
    (520, 300, 2, 101, 150, 640, 2.0, 0.0),      # band above the main diagonal, odd first offset
    (128, 64, 4, -63, 127, 256, 1.0, 0.0),       # every diagonal of a small matrix
])
def test_prod_steep_band_wide_batches(cb, trans, h, w, rf, lo, nd, ncols, fab, fc):
    """Bands with a row factor above 1 times many batch columns (the streaming banded kernel)."""
    rng = np.random.default_rng(h + 7 * nd + ncols + rf + (trans == "t"))
    offs = np.arange(lo, lo + nd, dtype=np.int32)
    prod_case(cb, rng, h, w, offs, rf, ncols, trans, fab, fc)


@pytest.mark.parametrize("trans", ["n", "t"])
@pytest.mark.parametrize("h,w,nd,spread,ncols,fab,fc", [
    (1500, 1404, 70, None, 40, 1.0, 0.0),       # ragged last row tile, 70 diagonals (not a multiple of 8), five column groups
    (1500, 1403, 70, None, 40, 1.5, 0.5),       # w not a multiple of 4: the last rows of a column are copied by hand
    (3000, 3000, 33, 600, 64, 1.0, 0.0),        # offsets within +-600: the small window (two blocks per SM)
    (2200, 2200, 1100, None, 32, 1.0, 0.0),     # more than 1024 diagonals: the variant that fetches its coefficients
    (700, 5000, 64, None, 36, 2.0, 1.0),        # much wider than tall: most of the window lies beyond the outputs' rows
    (8192, 8192, 100, 3000, 36, 1.0, 0.0),      # offsets within +-3000: a window of 6500 rows, four columns per block
    (4100, 4100, 48, 825, 40, 1.0, 0.0),        # a small window of 2107 / 2135 rows: its third segment is 59 / 87 rows long
])
def test_prod_scattered_staged_window(cb, trans, h, w, nd, spread, ncols, fab, fc):
    """Scattered diagonals with row factor 1 on operands that allow TMA (16-byte aligned, leading dimensions that are
    multiples of 4, NaN in the padding rows of B and in the padding cells of the diagonals): the staged-window kernels of
    prod_windown.cu, bit for bit against the host loop."""
    rng = np.random.default_rng(h + w + nd + (trans == "t"))
    lo, hi = (-spread, spread) if spread else (-h + 1, w - 1)
    offs = scattered_offsets(rng, nd, lo, hi, sort=(nd % 2 == 0))
    A = make_dia(rng, h, w, offs, 1, stride=(h + 3) // 4 * 4)
    rb, rc = (h, w) if trans == "t" else (w, h)
    B = F(rng.uniform(-1, 1, (rb, ncols)))
    C0 = F(rng.uniform(-1, 1, (rc, ncols)))
    if fc == 0:
        C0[:] = np.nan
    want = C0.copy(order="F")
    ho.prod(want, A, B, trans, fab, fc, nthreads=8)
    D = to_dev_dia(A)
    for mode in (cb.MODE_EXACT, cb.MODE_FAST):
        Cd = cb.to_device(C0)
        cb.prod(Cd, D, dev_padded(cb, B), trans, "n", fab, fc, mode)
        got = cb.to_host(Cd)
        if mode == cb.MODE_EXACT:
            assert_bits_equal(got, want, "staged-window prod %s" % trans)
        else:
            Aabs = ho.DiaHost(h, w, A.offsets, A.stride, 1, np.abs(np.nan_to_num(A.vals)))
            mag = F(np.abs(np.nan_to_num(C0)) * abs(fc))
            ho.prod(mag, Aabs, F(np.abs(B)), trans, abs(fab), 1.0, nthreads=8)
            assert np.all(np.abs(got.astype(np.float64) - want) <= 1e-5 * mag + 1e-30)
    assert cb.plan_status(D) == 0


def test_prod_staged_window_with_untouched_segments(cb):
    """Two clusters of diagonals far apart: the middle of the staged window is copied but touched by no term (the warp
    that issues the copies waits for them all the same)."""
    rng = np.random.default_rng(4242)
    h = w = 4096
    offs = np.concatenate([np.arange(-2040, -2040 + 3 * 11, 3), np.arange(2000, 2000 + 2 * 13, 2)]).astype(np.int32)
    prod_case(cb, rng, h, w, offs, 1, 48, "n", 1.0, 0.0)
    prod_case(cb, rng, h, w, offs, 1, 48, "t", 0.5, 2.0)


def test_prod_config0_shape(cb):
    """BASELINE config 0: 4096x4096, 64 sorted scattered diagonals, batch 128, factors 1/0."""
    rng = np.random.Generator(np.random.PCG64(1000))
    offs = scattered_offsets(rng, 64, -2047, 2047)
    prod_case(cb, rng, 4096, 4096, offs, 1, 128, "n", 1.0, 0.0)


def test_prod_config1_shape_reduced(cb):
    """BASELINE config 1 pattern (transposed, rf 4, band centred on 0, factC 0.5) at a quarter of the rows."""
    rng = np.random.Generator(np.random.PCG64(1001))
    offs = np.arange(-128, 128, dtype=np.int32)
    prod_case(cb, rng, 4096, 1024, offs, 4, 96, "t", 1.0, 0.5)


def test_prod_band_medium_both_ways(cb):
    """RBM-like band (config 3 pattern) at 2048 units, batch 160: up ('n') and down ('t')."""
    rng = np.random.Generator(np.random.PCG64(1003))
    offs = np.arange(-64, 64, dtype=np.int32)
    prod_case(cb, rng, 2048, 2048, offs, 1, 160, "n", 1.0, 0.0)
    prod_case(cb, rng, 2048, 2048, offs, 1, 160, "t", 1.0, 0.0)


@pytest.mark.parametrize("trans", ["n", "t"])
@pytest.mark.parametrize("n,nd,ncols", [(2048, 128, 96),      # tiled banded kernel
                                        (2048, 128, 1024),    # streaming banded kernel (wide batches)
                                        (65536, 12, 8),       # streaming kernel
                                        (4096, 40, 16)])      # run-walking kernel
def test_nonfinite_dense_values_beside_the_band(cb, trans, n, nd, ncols):
    """Inf and NaN in the dense operand.  Outputs whose band contains the bad row are non-finite in CUV's host loop
    (matrix_ops/spmv.cu:161-198) and here, with the same bits.  Outputs whose band lies well away from it are untouched
    in both.  In between lies the one stated deviation of the TMA-fed kernels: they walk the band in fixed-size
    chunks and give cells outside the band a zero coefficient instead of skipping them, so a non-finite dense value
    within a chunk's reach of the band (at most 64 rows here) turns the output into NaN where CUV would not read
    it.  The test pins exactly that: such outputs equal the oracle's or are NaN, nothing else."""
    rng = np.random.default_rng(n + nd)
    lo = -(nd // 2)
    A = make_dia(rng, n, n, np.arange(lo, lo + nd, dtype=np.int32), 1)
    B = F(rng.uniform(-1, 1, (n, ncols)))
    bad_rows = [n // 3, (2 * n) // 3 + 1]
    B[bad_rows[0], :] = np.inf
    B[bad_rows[1], :] = np.nan
    want = F(np.zeros((n, ncols)))
    ho.prod(want, A, B, trans, nthreads=4)
    got = run_prod(cb, A, B, F(np.zeros((n, ncols))), trans, 1.0, 0.0, cb.MODE_EXACT)
    out = np.arange(n)
    # output i reads dense rows i+lo .. i+lo+nd-1 ('n') or i-lo-nd+1 .. i-lo ('t')
    first = out + lo if trans == "n" else out - lo - nd + 1
    dist = np.full(n, 10 ** 9)
    for r in bad_rows:
        inside = (first <= r) & (r <= first + nd - 1)
        d = np.where(inside, 0, np.minimum(np.abs(first - r), np.abs(first + nd - 1 - r)))
        dist = np.minimum(dist, d)
    hit, far = dist == 0, dist > 64
    assert not np.isfinite(want[hit]).any() and np.isfinite(want[~hit]).all()
    assert_bits_equal(got[far], want[far], "outputs away from the non-finite rows")
    assert not np.isfinite(got[hit]).any()
    assert np.array_equal(np.isnan(got[hit]), np.isnan(want[hit]))
    assert_bits_equal(np.where(np.isnan(got[hit]), 0, got[hit]), np.where(np.isnan(want[hit]), 0, want[hit]), "inf outputs")
    near = ~hit & ~far
    same = (got[near].view(np.uint32) == want[near].view(np.uint32)) | ((got[near] == 0) & (want[near] == 0))
    assert np.all(same | np.isnan(got[near]))


def test_spmv_packed_vectors(cb):
    rng = np.random.default_rng(77)
    A = make_dia(rng, 64, 48, np.array([0, -3, 5], dtype=np.int32))
    v = rng.uniform(-1, 1, 48 * 3).astype(np.float32)
    D = to_dev_dia(A)
    dst = cb.to_device(np.zeros(64 * 3, dtype=np.float32))
    cb.spmv(dst, D, cb.to_device(v), "n", 2.0, 0.0)
    want = F(np.zeros((64, 3)))
    ho.prod(want, A, F(v.reshape(48, 3, order="F")), "n", 2.0, 0.0)
    assert_bits_equal(cb.to_host(dst).reshape(64, 3, order="F"), want)


def test_prod_preconditions(cb):
    rng = np.random.default_rng(1)
    A = make_dia(rng, 32, 16, np.arange(-3, 4, dtype=np.int32))
    D = to_dev_dia(A)
    B, C = cb.colmajor_empty(16, 6), cb.colmajor_empty(32, 6)
    with pytest.raises(cb.CuvDiaError, match="transB == 'n'"):
        cb.prod(C, D, B, "n", "t")
    with pytest.raises(cb.CuvDiaError):
        cb.prod(C, D, B, "x", "n")
    with pytest.raises(cb.CuvDiaError):
        cb.prod(C, D, cb.colmajor_empty(16, 5))
    with pytest.raises(cb.CuvDiaError):
        cb.prod(B, D, C, "n")                         # heights swapped
    with pytest.raises(cb.CuvDiaError, match="row_fact > 0"):
        cb.dev_dia_matrix_f(8, 8, [0], row_fact=0)


@pytest.mark.parametrize("trans", ["n", "t"])
def test_prod_with_repeated_offsets(cb, trans):
    """A diagonal number may occur in several slots (the reference's speed fixture stores each of its fs*fs
    offsets once per map, src/tests/spmv_speed.cpp:96-104): prod sums every stored diagonal."""
    rng = np.random.default_rng(21)
    px, fs, nm = 16, 3, 4
    h, w = px * px, 2 * px * px
    offs = np.array([i * px + j for _ in range(nm) for i in range(fs) for j in range(fs)], dtype=np.int32)
    A = make_dia(rng, h, w, offs, 1)
    rows_b, rows_c = (h, w) if trans == "t" else (w, h)
    B = np.asfortranarray(rng.standard_normal((rows_b, 14)).astype(np.float32))
    C0 = np.asfortranarray(rng.standard_normal((rows_c, 14)).astype(np.float32))
    want = C0.copy(order="F")
    ho.prod(want, A, B, trans, 2.0, 1.3)
    Cd = cb.to_device(C0)
    cb.prod(Cd, to_dev_dia(A), cb.to_device(B), trans, "n", 2.0, 1.3, cb.MODE_EXACT)
    assert_bits_equal(cb.to_host(Cd), want, "prod %s with repeated offsets" % trans)


def test_dd2dia_with_repeated_offsets(cb):
    """densedense_to_dia fills every slot, repeated diagonal numbers included; element access sees the last."""
    rng = np.random.default_rng(22)
    offs = np.array([0, 3, 0, -2, 3], dtype=np.int32)
    h = w = 96
    X = np.asfortranarray(rng.standard_normal((h, 40)).astype(np.float32))
    Y = np.asfortranarray(rng.standard_normal((w, 40)).astype(np.float32))
    ref = ho.DiaHost(h, w, offs, h, 1)
    ho.densedense_to_dia(ref, X, Y, 1.0, 0.0)
    D = cb.dev_dia_matrix_f(h, w, offs)
    D.vec.zero_()
    cb.densedense_to_dia(D, None, cb.to_device(X), cb.to_device(Y), 1.0, 0.0)
    got = D.vec.cpu().numpy()
    m = ref.valid_mask().reshape(-1)
    np.testing.assert_allclose(got[m], ref.vals[m], rtol=1e-4, atol=1e-5)
    assert np.array_equal(got[:h], got[2 * h:3 * h]) and D(5, 5) == got[2 * h + 5]


def dev_padded(cb, M):
    """Device copy of a column-major host matrix whose leading dimension is rounded up to a multiple of four (the
    padding rows hold NaN), as a view of its real rows: the 16-byte column alignment the vector kernels want."""
    rows, cols = M.shape
    buf = cb.colmajor_empty(rows + (4 - rows % 4) % 4, cols)
    buf.fill_(float("nan"))
    buf[:rows].copy_(cb.to_device(M))
    return buf[:rows]


def conv_offsets(px, py, fs, maps_in, maps_out):
    """Diagonal numbers of a convolution matrix as basics/filter_factory.hpp:58-76 builds them: per map block a run
    of fs diagonals per filter row, the next filter row one image line further, centred on the filter's middle."""
    offs = [i * px + j + m * px * py for m in range(maps_out + maps_in - 1) for i in range(fs) for j in range(fs)]
    return np.array(offs, dtype=np.int32) - (px + 1) * (fs // 2) - (maps_in - 1) * px * py


@pytest.mark.parametrize("trans", ["n", "t"])
@pytest.mark.parametrize("px,fs,mi,mo,ncols,fab,fc", [
    (16, 8, 1, 1, 14, 2.0, 1.3),        # one map, full passes of 8
    (16, 8, 1, 3, 14, 1.0, 0.0),        # three output maps: the matrix is three images wide
    (17, 5, 1, 2, 16, 0.5, 0.0),        # odd line length: every run has another alignment; runs shorter than a pass
    (12, 11, 2, 2, 33, 1.0, -1.0),      # runs of 11 = 8 + 3, two input maps (negative offsets), three column groups
    (20, 4, 1, 1, 1, 1.0, 0.0),         # spmv
])
def test_prod_convolution_pattern(cb, trans, px, fs, mi, mo, ncols, fab, fc):
    """Diagonals in runs (a convolution written as a DIA matrix) take the run-walking kernel; bit-exact against the
    host loop in EXACT mode, and within rounding of it in FAST mode."""
    rng = np.random.default_rng(px * 100 + fs)
    h, w = px * px * mi, px * px * mo
    offs = conv_offsets(px, px, fs, mi, mo)
    A = make_dia(rng, h, w, offs, 1)
    assert to_dev_dia(A).nnz > 0
    rows_b, rows_c = (h, w) if trans == "t" else (w, h)
    B = np.asfortranarray(rng.standard_normal((rows_b, ncols)).astype(np.float32))
    C0 = np.asfortranarray(rng.standard_normal((rows_c, ncols)).astype(np.float32))
    if fc == 0.0:
        C0[:] = np.nan                                 # factC == 0 must not read C
    want = C0.copy(order="F")
    ho.prod(want, A, B, trans, fab, fc)
    D = to_dev_dia(A)
    Cd = cb.to_device(C0)
    cb.prod(Cd, D, dev_padded(cb, B), trans, "n", fab, fc, cb.MODE_EXACT)
    assert_bits_equal(cb.to_host(Cd), want, "conv-pattern prod %s" % trans)
    Cd = cb.to_device(C0)
    cb.prod(Cd, D, dev_padded(cb, B), trans, "n", fab, fc, cb.MODE_FAST)
    scale = np.zeros_like(want)
    ho.prod(scale, ho.DiaHost(A.h, A.w, A.offsets, A.stride, 1, np.abs(np.nan_to_num(A.vals))), np.abs(B), trans, abs(fab), 0.0)
    assert np.all(np.abs(cb.to_host(Cd) - want) <= 1e-5 * (scale + np.abs(np.nan_to_num(C0) * fc)) + 1e-30)


@pytest.mark.parametrize("trans", ["n", "t"])
def test_prod_runs_ragged_and_repeated(cb, trans):
    """Runs on a matrix whose sizes are not multiples of four, wider than tall, with one run stored twice and a
    single stray diagonal between runs."""
    rng = np.random.default_rng(77)
    h, w = 203, 517
    offs = np.concatenate([np.arange(-9, -1), np.arange(40, 52), [300], np.arange(40, 48), np.arange(100, 109),
                           np.arange(-203, -195), np.arange(509, 517)]).astype(np.int32)
    A = make_dia(rng, h, w, offs, 1, stride=208)
    rows_b, rows_c = (h, w) if trans == "t" else (w, h)
    B = np.asfortranarray(rng.standard_normal((rows_b, 19)).astype(np.float32))
    C0 = np.asfortranarray(rng.standard_normal((rows_c, 19)).astype(np.float32))
    want = C0.copy(order="F")
    ho.prod(want, A, B, trans, 1.5, 0.25)
    Cd = cb.to_device(C0)
    cb.prod(Cd, to_dev_dia(A), dev_padded(cb, B), trans, "n", 1.5, 0.25, cb.MODE_EXACT)
    assert_bits_equal(cb.to_host(Cd), want, "runs, ragged %s" % trans)


# ---- densedense_to_dia -------------------------------------------------------------------------------

def dd_case(cb, rng, h, w, offsets, rf, ncols, fab, fc, stride=None, dist="rbm", addend_scale=False):
    """One densedense_to_dia call against the host loop.  addend_scale: where factC * C_old and factAB * sum nearly
    cancel, no summation order can promise an error relative to the small result; such cells are also accepted within
    a few units in the last place of the addends' magnitudes."""
    C = make_dia(rng, h, w, offsets, rf, stride)
    if dist == "rbm":
        X = F((rng.uniform(0, 1, (h, ncols)) < 0.5).astype(np.float32))
        H = F(1.0 / (1.0 + np.exp(-rng.standard_normal((w, ncols)))))
    else:
        X, H = F(rng.uniform(0, 1, (h, ncols))), F(rng.uniform(0, 1, (w, ncols)))
    want = ho.DiaHost(h, w, C.offsets, C.stride, rf, C.vals.copy())
    if fc == 0:
        C.vals[C.valid_mask().reshape(-1)] = np.nan      # old values must not be read
    ho.densedense_to_dia(want, X, H, fab, fc, nthreads=4)
    D = to_dev_dia(C)
    Xd, Hd = cb.to_device(X), cb.to_device(H)
    bd = cb.dev_block_descriptor_f(D)
    cb.densedense_to_dia(D, bd, Xd, Hd, fab, fc)
    got = D.vec.cpu().numpy()
    m = C.valid_mask().reshape(-1)
    assert_bits_equal(got[~m], C.vals[~m], "cells outside the diagonals' ranges must be untouched")
    tol = 1e-4 * np.sqrt(max(ncols, 128) / 128.0)
    if addend_scale:
        mag = ho.DiaHost(h, w, C.offsets, C.stride, rf, np.abs(np.nan_to_num(C.vals)))
        ho.densedense_to_dia(mag, np.abs(X), np.abs(H), abs(fab), abs(fc), nthreads=4)
        err = np.abs(got[m] - want.vals[m])
        assert np.all(err <= tol * np.abs(want.vals[m]) + 8 * 2.0 ** -24 * mag.vals[m])
    else:
        np.testing.assert_allclose(got[m], want.vals[m], rtol=tol, atol=tol * 1e-3)
    D2 = to_dev_dia(C)
    cb.densedense_to_dia(D2, bd, Xd, Hd, fab, fc)
    assert_bits_equal(D2.vec.cpu().numpy()[m], got[m], "run-to-run reproducibility")


@pytest.mark.parametrize("rf,h,w,nd,ncols,fab,fc", [
    (1, 1000, 1000, 70, 96, 1.0, 0.0),        # three groups of neighbours, the last one partial; ragged rows
    (1, 517, 900, 33, 100, 0.01, 0.9),        # wider than tall, batch not a multiple of the staged chunk
    (2, 1024, 700, 40, 64, -0.5, 1.0),        # row factor 2: two rows share a row of the second operand
    (4, 2048, 600, 64, 256, 1.0, 0.0),
])
def test_dd2dia_scattered_windowed(cb, rf, h, w, nd, ncols, fab, fc):
    """Scattered offsets whose neighbours (in offset order) lie close enough for the staged-window kernel: unsorted
    storage order, offsets reaching outside the matrix on both sides, every row factor."""
    rng = np.random.default_rng(300 + rf + nd)
    offs = scattered_offsets(rng, nd, -(h // rf) + 1, w - 1, sort=False)
    dd_case(cb, rng, h, w, offs, rf, ncols, fab, fc)


@pytest.mark.parametrize("h,w,ncols", [(4096, 4096, 200), (2500, 3000, 70)])
def test_dd2dia_scattered_groups_outside_the_matrix(cb, h, w, ncols):
    """Tiles of 512 rows and offsets spread over the whole matrix: for most tiles some of the diagonals lie wholly
    outside the matrix and are never scheduled, the groups of neighbours start at a different diagonal for every tile,
    and two clusters of offsets far apart cut a group short.  Every cell inside the matrix still gets its sum, every
    other cell stays as it was."""
    rng = np.random.default_rng(h + ncols)
    spread = scattered_offsets(rng, 96, -h + 1, w - 1, sort=False)
    clusters = np.concatenate([np.arange(-1500, -1500 + 3 * 7, 3), np.arange(900, 900 + 2 * 9, 2)]).astype(np.int32)
    offs = np.unique(np.concatenate([spread, clusters])).astype(np.int32)
    rng.shuffle(offs)
    dd_case(cb, rng, h, w, offs, 1, ncols, 0.01, 0.9, addend_scale=True)
    dd_case(cb, rng, h, w, offs, 1, ncols, 1.0, 0.0, dist="uniform")


@pytest.mark.parametrize("rf,h,w,lo,nd,ncols,fab,fc", [
    (4, 2048, 512, -64, 128, 200, 1.0, 0.0),       # config 1's pattern at an eighth of the size: one and a bit tiles per row block
    (2, 1024, 600, -50, 100, 96, 0.01, 0.9),       # row factor 2, both factors, batch not a multiple of the staged chunk
    (8, 4096, 512, -31, 200, 64, -0.5, 1.0),       # row factor 8, odd first offset
    (4, 1020, 300, 7, 64, 130, 1.0, 0.0),          # height not a multiple of the tile, band above the diagonal
    (32, 4096, 128, -60, 120, 64, 1.0, 0.0),       # the largest row factor the tiles take
])
def test_dd2dia_steep_band(cb, rf, h, w, lo, nd, ncols, fab, fc):
    """Bands with a row factor above 1 (cell (i, k) meets row i / rf + lo + k of the second operand) on the tiled kernel."""
    rng = np.random.default_rng(h + 7 * nd + rf)
    offs = np.arange(lo, lo + nd, dtype=np.int32)
    dd_case(cb, rng, h, w, offs, rf, ncols, fab, fc, addend_scale=(fc != 0))


def test_dd2dia_convolution_pattern(cb):
    """The weight gradient of a convolution-pattern matrix (runs of consecutive diagonals one image line apart,
    two input and two output maps): neighbouring runs share the staged window."""
    rng = np.random.default_rng(41)
    px, fs = 16, 5
    h, w = px * px * 2, px * px * 2
    offs = conv_offsets(px, px, fs, 2, 2)
    dd_case(cb, rng, h, w, offs, 1, 72, 1.0 / 72, 0.0)
    dd_case(cb, rng, h, w, offs, 1, 72, -1.0 / 72, 1.0, dist="uniform")


def test_dd2dia_runs_of_diagonals(cb):
    """Runs of consecutive diagonals as narrow bands of their own (the run-aware kernel): the reference's speed fixture
    (src/tests/densedense_to_dia_speed.cpp:65-106: a 28 x 28 image, 8 x 8 filters, two output maps whose diagonal numbers
    repeat), runs of unequal length with every alignment of their first offset, several row tiles with a ragged end,
    and both factors."""
    rng = np.random.default_rng(43)
    offs = np.array([i * 28 + j for _ in range(2) for i in range(8) for j in range(8)], dtype=np.int32)
    dd_case(cb, rng, 784, 1568, offs, 1, 96, 1.0, 0.0)
    runs = [(-301, 8), (-150, 7), (-9, 8), (2, 5), (43, 8), (60, 8), (201, 6), (350, 8), (-1290, 8), (1301, 8), (-37, 8),
            (500, 8), (521, 4), (-700, 8), (-650, 8), (777, 8)]
    offs = np.concatenate([np.arange(lo, lo + n) for lo, n in runs]).astype(np.int32)
    dd_case(cb, rng, 1300, 1411, offs, 1, 37, -0.5, 1.0, dist="uniform")
    dd_case(cb, rng, 1300, 1411, offs, 1, 16, 2.0, 0.0)


def test_reference_fixture_dd2dia(cb, golden):
    g = golden                                           # src/tests/densedense_to_dia.cpp:109-137,166-197
    h, w, rf, S = int(g["dd2dia_h"]), int(g["dd2dia_w"]), int(g["dd2dia_rf"]), int(g["dd2dia_stride"])
    D = cb.dev_dia_matrix_f(h, w, g["dd2dia_offsets"], S, rf)
    D.vec.zero_()
    cb.densedense_to_dia(D, cb.dev_block_descriptor_f(D), cb.to_device(g["dd2dia_A"]), cb.to_device(g["dd2dia_B"]))
    assert np.array_equal(D.vec.cpu().numpy().astype(np.float64), g["dd2dia_expect"])


@pytest.mark.parametrize("rf", [1, 2, 4])
def test_dd2dia_scattered_small(cb, rf):
    rng = np.random.default_rng(200 + rf)
    w, h = 150, 60 * rf
    offs = scattered_offsets(rng, 11, -(h // rf) + 1, w - 1, sort=False)
    dd_case(cb, rng, h, w, offs, rf, 48, 1.0, 0.0, stride=h + 4)
    dd_case(cb, rng, h, w, offs, rf, 200, 0.01, 0.9, dist="uniform")
    dd_case(cb, rng, h, w, offs, rf, 1, -0.5, 1.0)


@pytest.mark.parametrize("rf", [1, 2, 4])
@pytest.mark.parametrize("lo,nd", [(-8, 16), (-5, 11), (3, 40), (-70, 133)])
def test_dd2dia_band_small(cb, rf, lo, nd):
    rng = np.random.default_rng(300 + rf + nd)
    w, h = 200, 64 * rf
    offs = np.arange(lo, lo + nd, dtype=np.int32)
    dd_case(cb, rng, h, w, offs, rf, 96, 1.0, 0.0)
    dd_case(cb, rng, h, w, offs, rf, 130, 0.01, 0.9, stride=h + 8)


def test_dd2dia_config2_shape(cb):
    """BASELINE config 2: 4096x4096, 128 sorted scattered diagonals, batch 1024, 0.01 / 0.9."""
    rng = np.random.Generator(np.random.PCG64(1002))
    offs = scattered_offsets(rng, 128, -2047, 2047)
    dd_case(cb, rng, 4096, 4096, offs, 1, 1024, 0.01, 0.9)


def test_dd2dia_band_medium(cb):
    rng = np.random.Generator(np.random.PCG64(1013))
    dd_case(cb, rng, 2048, 2048, np.arange(-64, 64, dtype=np.int32), 1, 256, 1.0 / 256, 0.0)
    dd_case(cb, rng, 1000, 1100, np.arange(-30, 45, dtype=np.int32), 1, 77, 1.0, 1.0)


def test_dd2dia_preconditions(cb):
    D = cb.dev_dia_matrix_f(30, 16, [0, 1], row_fact=4)           # 30 % 4 != 0
    with pytest.raises(cb.CuvDiaError, match="rf == 0"):
        cb.densedense_to_dia(D, None, cb.colmajor_empty(30, 4), cb.colmajor_empty(16, 4))
    D = cb.dev_dia_matrix_f(32, 16, [0, 1])
    with pytest.raises(cb.CuvDiaError):
        cb.densedense_to_dia(D, None, cb.colmajor_empty(32, 4), cb.colmajor_empty(16, 5))


# ---- reductions ----------------------------------------------------------------------------------------

ALL_RF = [ho.RF_ADD, ho.RF_MEAN, ho.RF_ADD_SQUARED, ho.RF_MAX, ho.RF_ARGMAX, ho.RF_ARGMIN, ho.RF_MIN, ho.RF_MULT,
          ho.RF_LOGADDEXP, ho.RF_ADDEXP]


def reduce_case(cb, rng, rows, cols, to_col, rf, fnew=1.0, fold=0.0, row_major=False):
    import torch
    lo = 0.5 if rf == ho.RF_MULT else -1.0
    src = F(rng.uniform(lo, 1.5, (rows, cols)))
    n_out = rows if to_col else cols
    old = rng.standard_normal(n_out).astype(np.float32)
    want = old.copy() if fold != 0 else np.full(n_out, np.nan, dtype=np.float32)
    (ho.reduce_to_col if to_col else ho.reduce_to_row)(want, src, rf, fnew, fold, nthreads=4)
    dsrc = torch.from_numpy(np.ascontiguousarray(src)).cuda() if row_major else cb.to_device(src)
    dst = cb.to_device(old if fold != 0 else np.full(n_out, np.nan, dtype=np.float32))
    (cb.reduce_to_col if to_col else cb.reduce_to_row)(dst, dsrc, rf, fnew, fold)
    got = dst.cpu().numpy()
    if rf in (ho.RF_MAX, ho.RF_MIN, ho.RF_ARGMAX, ho.RF_ARGMIN):
        assert np.array_equal(got, want)
    else:
        n_red = cols if to_col else rows
        tol = 1e-4 * np.sqrt(max(n_red, 128) / 128.0)
        np.testing.assert_allclose(got, want, rtol=tol, atol=tol * 1e-2)


@pytest.mark.parametrize("rf", ALL_RF)
@pytest.mark.parametrize("to_col", [True, False])
@pytest.mark.parametrize("row_major", [False, True])
def test_reduce_reference_sweep(cb, rf, to_col, row_major):
    """The shape of the reference's sweep (src/tests/matrix_op.cpp:858-924): 270x270, both axes, both layouts."""
    rng = np.random.default_rng(rf * 4 + to_col * 2 + row_major)
    reduce_case(cb, rng, 270, 270, to_col, rf, row_major=row_major)


@pytest.mark.parametrize("to_col", [True, False])
def test_reduce_shapes_and_factors(cb, to_col):
    rng = np.random.default_rng(55 + to_col)
    for rows, cols in [(1, 1), (1, 300), (300, 1), (4096, 96), (96, 4096), (33, 70001), (70001, 33), (2048, 2048),
                       (32, 65536), (65536, 32), (8, 100000), (100000, 8), (256, 5000), (64, 8192), (16, 4100)]:
        reduce_case(cb, rng, rows, cols, to_col, ho.RF_ADD, 0.25, 0.5)
        reduce_case(cb, rng, rows, cols, to_col, ho.RF_ARGMAX)
    reduce_case(cb, rng, 16384, 256, to_col, ho.RF_ADD, 1.0 / 256, 1.0)


def test_reduce_ties_take_first_index(cb):
    import torch
    src = np.zeros((64, 5000), dtype=np.float32, order="F")
    src[:, 17] = 3.0; src[:, 4000] = 3.0
    dst = torch.empty(64, device="cuda")
    cb.reduce_to_col(dst, cb.to_device(src), ho.RF_ARGMAX)
    assert np.array_equal(dst.cpu().numpy(), np.full(64, 17.0, dtype=np.float32))
    srcT = np.asfortranarray(src.T)
    dst = torch.empty(64, device="cuda")
    cb.reduce_to_row(dst, cb.to_device(srcT), ho.RF_ARGMAX)
    assert np.array_equal(dst.cpu().numpy(), np.full(64, 17.0, dtype=np.float32))


def test_reduce_preconditions(cb):
    import torch
    src = cb.colmajor_empty(8, 4)
    with pytest.raises(cb.CuvDiaError):
        cb.reduce_to_col(torch.empty(4, device="cuda"), src)
    with pytest.raises(cb.CuvDiaError, match="factNew == 1"):
        cb.reduce_to_col(torch.empty(8, device="cuda"), src, ho.RF_MEAN, 2.0, 0.0)


# ---- glue ------------------------------------------------------------------------------------------------

@pytest.mark.parametrize("units,ncols", [(64, 8), (37, 5), (4096, 33)])
def test_bias_sigmoid_sample(cb, units, ncols):
    rng = np.random.default_rng(units)
    a = F(rng.standard_normal((units, ncols)) * 3)
    b = rng.standard_normal(units).astype(np.float32)
    p = a.copy(order="F")
    ho.bias_sigmoid_sample(p, b, None)
    u = F(rng.uniform(0, 1, (units, ncols)))
    near = np.abs(p - u) < 1e-4                         # keep the compare away from ties (expf differs by ulps)
    u[near] = np.where(p[near] > 0.5, 0.0, 1.0)
    s_want = (p > u).astype(np.float32)
    ad = cb.to_device(a)
    sd = cb.bias_sigmoid_sample(ad, cb.to_device(b), cb.to_device(u))
    np.testing.assert_allclose(cb.to_host(ad), p, rtol=1e-5)
    assert np.array_equal(cb.to_host(sd), s_want)
    ad = cb.to_device(a)
    assert cb.bias_sigmoid_sample(ad) is None
    q = a.copy(order="F"); ho.bias_sigmoid_sample(q, None, None)
    np.testing.assert_allclose(cb.to_host(ad), q, rtol=1e-5)


def test_axpby(cb):
    rng = np.random.default_rng(4)
    x, y = rng.standard_normal(1001).astype(np.float32), rng.standard_normal(1001).astype(np.float32)
    xd, yd = cb.to_device(x), cb.to_device(y)
    cb.axpby(xd, xd, yd, 0.9, -0.01)
    assert_bits_equal(xd.cpu().numpy(), np.float32(0.9) * x + np.float32(-0.01) * y)


@pytest.mark.parametrize("n,skip", [(1, 0), (1001, 0), (4096, 0), (70001, 1), (1 << 20, 3)])
@pytest.mark.parametrize("lr,decay", [(0.01, 0.0), (0.1, 0.05), (1.0, 0.05)])
def test_learn_step_weight_decay(cb, n, skip, lr, decay):
    """W = -lr*dW + (1 - lr*decay)*W, bit for bit with the host loop (tensor_ops/rprop.cu:331-346), at sizes that are
    not a multiple of four and from pointers that are not 16-byte aligned; 1.f/0.05f is tensor_op_speed.cpp:177."""
    import torch
    rng = np.random.default_rng(n + skip)
    w, g = rng.standard_normal(n + skip).astype(np.float32), rng.standard_normal(n + skip).astype(np.float32)
    wd, gd = cb.to_device(w), cb.to_device(g)
    cb.learn_step_weight_decay(wd[skip:], gd[skip:], lr, decay)
    torch.cuda.synchronize()
    ref = w.copy()
    ho.learn_step_weight_decay(ref[skip:], g[skip:], lr, decay)
    assert_bits_equal(wd.cpu().numpy(), ref)


@pytest.mark.parametrize("n,skip", [(1001, 0), (70001, 1), (1 << 18, 0)])
def test_learn_step_weight_decay_momentum(cb, n, skip):
    """The momentum step with the device kernel's formula (tensor_ops/rprop.cu:158-170), three steps in a row."""
    import torch
    rng = np.random.default_rng(n)
    w, g, m = (rng.standard_normal(n + skip).astype(np.float32) for _ in range(3))
    wd, gd, md = cb.to_device(w), cb.to_device(g), cb.to_device(m)
    wr, mr = w.copy(), m.copy()
    for it in range(3):
        cb.learn_step_weight_decay_momentum(wd[skip:], md[skip:], gd[skip:], 0.01, 0.9 - 0.1 * it, 0.002)
        ho.learn_step_weight_decay_momentum(wr[skip:], mr[skip:], g[skip:], 0.01, 0.9 - 0.1 * it, 0.002)
    torch.cuda.synchronize()
    assert_bits_equal(wd.cpu().numpy(), wr)
    assert_bits_equal(md.cpu().numpy(), mr)


def test_learn_step_on_dia_matrix(cb):
    """The sparse RBM's update (examples/rbm/base.py:72-73): the step over a DIA matrix's whole value array."""
    offs = np.arange(-3, 4, dtype=np.int32)
    W = cb.dev_dia_matrix_f(200, 200, offs)
    G = cb.dev_dia_matrix_f(200, 200, offs)
    rng = np.random.default_rng(5)
    w, g = rng.standard_normal(W.vec.numel()).astype(np.float32), rng.standard_normal(W.vec.numel()).astype(np.float32)
    W.set_vec(w); G.set_vec(g)
    cb.learn_step_weight_decay(W, G, 0.05, 0.01)
    ref = w.copy()
    ho.learn_step_weight_decay(ref, g, 0.05, 0.01)
    assert_bits_equal(W.vec.cpu().numpy(), ref)
    with pytest.raises(cb.CuvDiaError):
        cb.learn_step_weight_decay(W, G.vec[:-1], 0.05)


def test_convert_and_pull(cb, golden):
    """dia_mat.cpp:111-132 / convert.cpp:110-129 on the Python mirror: host -> device -> host round trip and
    dia -> dense equal the reference fixture."""
    g = golden
    H = cb.host_dia_matrix_f(int(g["diamat_h"]), int(g["diamat_w"]), g["diamat_offsets"], int(g["diamat_stride"]))
    H.vec[:] = g["diamat_vals"]
    D = cb.dev_dia_matrix_f(int(g["diamat_h"]), int(g["diamat_w"]), g["diamat_offsets"], int(g["diamat_stride"]))
    cb.convert(D, H)
    H2 = cb.host_dia_matrix_f(1, 1, [0])
    cb.convert(H2, D)
    assert np.array_equal(H2.vec, H.vec) and np.array_equal(H2.offsets, H.offsets)
    assert np.array_equal(cb.convert(None, H), g["diamat_dense"])
    assert np.array_equal(cb.pull(D), g["diamat_dense"])
    assert D(3, 4) == H(3, 4) == g["diamat_dense"][3, 4] and not H.has(0, 5)


@pytest.mark.parametrize("trans", ["n", "t"])
@pytest.mark.parametrize("lo,nd", [(-8, 16), (-5, 11), (3, 16), (-2, 5), (1, 16)])
def test_prod_streaming_narrow_band(cb, trans, lo, nd):
    """Long, narrow bands (the TMA streaming kernel: >= 32768 rows, <= 16 diagonals), all four alignments of the
    first offset, ragged row counts, more than 32 columns, factC != 0."""
    rng = np.random.default_rng(900 + nd + 31 * (trans == "t") + lo)
    offs = np.arange(lo, lo + nd, dtype=np.int32)
    prod_case(cb, rng, 40004, 36008, offs, 1, 5, trans, 1.0, 0.0)
    prod_case(cb, rng, 36008, 40004, offs, 1, 40, trans, 0.75, 2.0)


def test_spmv_long_tridiagonal(cb):
    """The classical DIA use: a tridiagonal operator times one vector, through spmv."""
    rng = np.random.default_rng(17)
    n = 1 << 17
    A = make_dia(rng, n, n, np.array([-1, 0, 1], dtype=np.int32))
    v = rng.uniform(-1, 1, n).astype(np.float32)
    D = to_dev_dia(A)
    dst = cb.to_device(np.zeros(n, dtype=np.float32))
    cb.spmv(dst, D, cb.to_device(v), "n")
    want = F(np.zeros((n, 1)))
    ho.prod(want, A, F(v.reshape(n, 1)), "n")
    assert_bits_equal(cb.to_host(dst), want[:, 0])


@pytest.mark.parametrize("lo,nd", [(-8, 16), (-5, 11), (3, 16), (-2, 5), (1, 16)])
def test_dd2dia_streaming_narrow_band(cb, lo, nd):
    """Long, narrow bands (the TMA streaming densedense_to_dia: >= 32768 rows, <= 16 diagonals): all alignments
    of the first offset, ragged sizes, batch not a multiple of the round, both factor paths."""
    rng = np.random.default_rng(950 + nd + lo)
    offs = np.arange(lo, lo + nd, dtype=np.int32)
    dd_case(cb, rng, 40004, 36008, offs, 1, 40, 1.0, 0.0)
    dd_case(cb, rng, 36008, 40004, offs, 1, 21, 0.01, 0.9, dist="uniform")


def test_avg_diagonals(cb):
    """Mean of every stored diagonal over its cells inside the matrix (host definition, matrix_ops/diagonals.cu:23-48):
    padding cells (NaN here) never enter; unsorted offsets; tall, wide and large matrices."""
    import torch
    rng = np.random.default_rng(11)
    for h, w, offs in [(32, 16, [0, 1, -1]), (57, 150, [5, -40, 149, 0, -56]), (4096, 4096, list(range(-70, 58)))]:
        A = make_dia(rng, h, w, np.array(offs, dtype=np.int32), 1)
        want = np.zeros(len(offs), dtype=np.float32)
        ho.avg_diagonals(want, A)
        got = torch.full((len(offs),), 7.0, device="cuda")
        cb.avg_diagonals(got, to_dev_dia(A))
        np.testing.assert_allclose(got.cpu().numpy(), want, rtol=1e-4, atol=1e-6)
    # the dia_mat.cpp fixture (src/tests/dia_mat.cpp:134-142 with the call restored): diagonal k of a matrix filled with k
    A = ho.DiaHost(32, 16, np.array([0, 1, -1], dtype=np.int32), 32, 1)
    A.vals[:] = np.repeat(np.array([3.0, 5.0, -2.0], dtype=np.float32), 32)
    got = torch.empty(3, device="cuda")
    cb.avg_diagonals(got, to_dev_dia(A))
    assert got.cpu().numpy().tolist() == [3.0, 5.0, -2.0]
    with pytest.raises(cb.CuvDiaError):
        cb.avg_diagonals(got, to_dev_dia(make_dia(rng, 32, 16, np.array([0, 1, -1], dtype=np.int32), 2)))


TYPED_PAIRS = [("int32", "float32"), ("uint32", "float32"), ("uint8", "float32"), ("float32", "int32"),
               ("float32", "uint32"), ("float32", "uint8"), ("uint8", "uint8"), ("uint8", "uint32")]


def typed_source(rng, dtype, shape, small):
    """Values for which C++ defines every conversion of CUV's host loop and every sum stays exact in float (below
    2^24): non-negative, and small where they are squared or summed through an 8-bit value."""
    if dtype == "uint8":
        return np.asfortranarray(rng.integers(0, 3 if small else 256, shape).astype(np.uint8))
    if dtype == "int32":
        return np.asfortranarray(rng.integers(-50, 50, shape).astype(np.int32) if small else
                                 rng.integers(-1000, 1000, shape).astype(np.int32))
    if dtype == "uint32":
        return np.asfortranarray(rng.integers(0, 60 if small else 3000, shape).astype(np.uint32))
    return np.asfortranarray((rng.uniform(0, 2.99 if small else 200.0, shape)).astype(np.float32))


@pytest.mark.parametrize("src_t,dst_t", TYPED_PAIRS)
@pytest.mark.parametrize("shape", [(270, 33), (37, 4100), (1030, 1030)])
def test_reduce_between_element_types(cb, src_t, dst_t, shape):
    """The eight other (source, destination) pairs CUV instantiates (matrix_ops/matrix_ops_reduce.cu:395-413), both
    axes, bit for bit against the restated host loop: running value in the source type, fold in the destination type,
    factors converted to the source type, indices for the arg forms."""
    import torch
    import zlib
    rng = np.random.default_rng(zlib.crc32(("%s %s %s" % (src_t, dst_t, shape)).encode()))
    tdt = {"float32": torch.float32, "int32": torch.int32, "uint32": torch.uint32, "uint8": torch.uint8}
    cases = [(ho.RF_ADD, 1.0, 0.0, True), (ho.RF_ADD, 2.0, 3.0, True), (ho.RF_MEAN, 1.0, 0.0, True),
             (ho.RF_ADD_SQUARED, 1.0, 0.0, True), (ho.RF_MAX, 1.0, 0.0, False), (ho.RF_MIN, 1.0, 1.0, False),
             (ho.RF_ARGMAX, 1.0, 0.0, False), (ho.RF_ARGMIN, 1.0, 0.0, False)]
    for rf, fn, fo, summed in cases:
        # sums that travel through an 8-bit value must stay below 256 for the host loop to be defined
        eight_bit = summed and ("uint8" in (src_t, dst_t))
        for over_strided in (True, False):
            n_red = shape[1] if over_strided else shape[0]
            small = eight_bit or rf == ho.RF_ADD_SQUARED
            src = typed_source(rng, src_t, shape, small)
            if eight_bit:
                # keep each line's total (and factNew * total + factOld * old) inside 8 bits: about 20 non-zero
                # elements of at most 2 per line
                keep = rng.random(shape) < min(1.0, 20.0 / n_red)
                src = np.asfortranarray(np.where(keep, src, 0).astype(src.dtype))
            n_out = shape[0] if over_strided else shape[1]
            old = rng.integers(0, 3, n_out).astype(dst_t)
            want = old.copy()
            ho.reduce_typed(want, src, over_strided, rf, fn, fo)
            dsrc = torch.from_numpy(np.ascontiguousarray(src.T)).cuda().t()
            ddst = torch.from_numpy(old.copy()).cuda()
            assert ddst.dtype == tdt[dst_t]
            (cb.reduce_to_col if over_strided else cb.reduce_to_row)(ddst, dsrc, rf, fn, fo)
            got = ddst.cpu().numpy()
            assert np.array_equal(got, want), "%s -> %s rf=%d over_strided=%s: %d of %d differ" % (
                src_t, dst_t, rf, over_strided, int((got != want).sum()), got.size)


def test_reduce_element_type_errors(cb):
    import torch
    src = torch.zeros((8, 8), dtype=torch.int32, device="cuda").t()
    with pytest.raises(cb.CuvDiaError, match="no instantiation"):
        cb.reduce_to_col(torch.zeros(8, dtype=torch.int32, device="cuda"), src)
    with pytest.raises(cb.CuvDiaError, match="float -> float only"):
        cb.reduce_to_col(torch.zeros(8, dtype=torch.float32, device="cuda"), src, cb.RF_LOGADDEXP)


def test_bounded_wait_gives_up_with_a_status(cb):
    """A wait that nothing will ever satisfy runs out after its poll limit, leaves a code in the plan's health word
    and returns; the device stays usable (the next product is bit-exact) and the word can be cleared."""
    import ctypes
    import torch
    from cuv_b200 import _capi
    L = _capi.lib()
    rng = np.random.default_rng(5)
    A = make_dia(rng, 300, 300, np.arange(-20, 20, dtype=np.int32), 1, stride=304)
    D = to_dev_dia(A)
    st = ctypes.c_int(-1)
    _capi.check(L.cuvdia_plan_status(D._plan, ctypes.byref(st)))
    assert st.value == 0
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    _capi.check(L.cuvdia_selftest_bounded_wait(D._plan, 2000, stream))
    _capi.check(L.cuvdia_plan_status(D._plan, ctypes.byref(st)))
    assert st.value == 9
    assert L.cuvdia_selftest_bounded_wait(D._plan, 0, stream) == _capi.ERR_INVALID
    B = np.asfortranarray(rng.standard_normal((300, 70)).astype(np.float32))
    want = np.zeros((300, 70), dtype=np.float32, order="F")
    ho.prod(want, A, B, "n")
    C = cb.colmajor_empty(300, 70)
    # the blocking form of a call notices the code, clears it and raises, as CUV throws from a failed operation
    with pytest.raises(cb.CuvDiaError, match="gave up a bounded wait"):
        cb.prod(C, D, dev_padded(cb, B), "n", "n", 1.0, 0.0, cb.MODE_EXACT, check_status=True)
    assert cb.plan_status(D) == 0
    _capi.check(L.cuvdia_selftest_bounded_wait(D._plan, 2000, stream))
    with pytest.raises(cb.CuvDiaError, match="gave up a bounded wait"):
        cb.densedense_to_dia(D, None, cb.colmajor_empty(300, 8).zero_(), cb.colmajor_empty(300, 8).zero_(), 1.0, 1.0,
                             check_status=True)
    D.set_vec(A.vals)
    cb.prod(C, D, dev_padded(cb, B), "n", "n", 1.0, 0.0, cb.MODE_EXACT, check_status=True)
    assert_bits_equal(cb.to_host(C), want, "prod after the self-test")
    _capi.check(L.cuvdia_plan_status(D._plan, ctypes.byref(st)))
    assert st.value == 0
