"""Seeded random sweep over shapes, diagonal patterns, row factors, batch sizes, factors and operand
alignments: whatever kernel the dispatcher picks, prod must reproduce the host loop bit for bit in the EXACT
arithmetic and densedense_to_dia must stay within the gradient tolerance and leave padding cells untouched."""
import os

import numpy as np
import pytest

from oracle import host_oracle as ho
from tests.helpers import F, assert_bits_equal, make_dia, to_dev_dia

pytestmark = pytest.mark.gpu

# more seeds for an occasional longer hunt: CUVDIA_FUZZ_SCALE=10 runs ten times as many cases
SCALE = int(os.environ.get("CUVDIA_FUZZ_SCALE", "1"))


@pytest.fixture(scope="module")
def cb():
    import cuv_b200
    return cuv_b200


def random_offsets(rng, h, w, rf):
    """One of the pattern classes the plan distinguishes: a band, runs of consecutive diagonals (a convolution
    pattern), scattered offsets, scattered offsets with repeats; in storage order that is sorted or shuffled."""
    lo_min, hi_max = -(h // rf) + 1, w - 1
    span = hi_max - lo_min + 1
    kind = rng.integers(0, 4)
    if kind == 0:                                             # band
        nd = int(rng.integers(1, min(80, span) + 1))
        lo = int(rng.integers(lo_min, hi_max - nd + 2))
        offs = np.arange(lo, lo + nd)
    elif kind == 1:                                           # runs
        runs, fs, step = int(rng.integers(2, 7)), int(rng.integers(3, 13)), int(rng.integers(13, 60))
        lo = int(rng.integers(lo_min, max(lo_min + 1, hi_max - runs * step - fs)))
        offs = np.concatenate([lo + r * step + np.arange(fs) for r in range(runs)])
        offs = offs[(offs >= lo_min) & (offs <= hi_max)]
        if offs.size == 0:
            offs = np.array([0])
        if rng.integers(0, 3) == 0:                           # the same runs stored twice, as the speed fixture does
            offs = np.concatenate([offs, offs])
    else:                                                     # scattered
        nd = int(rng.integers(1, min(70, span) + 1))
        offs = rng.choice(np.arange(lo_min, hi_max + 1), nd, replace=False)
        offs = np.sort(offs) if rng.integers(0, 2) else offs
        if kind == 3 and nd > 2:
            offs[int(rng.integers(0, nd))] = offs[int(rng.integers(0, nd))]
    return offs.astype(np.int32)


def device_matrix(cb, rng, M, pad):
    """Device copy of a column-major host matrix; with ``pad`` the leading dimension is rounded up to a multiple of
    four (NaN in the padding rows) so that the vector kernels qualify, without it they do not when rows % 4 != 0."""
    if not pad:
        return cb.to_device(M)
    rows, cols = M.shape
    buf = cb.colmajor_empty(rows + (4 - rows % 4) % 4, cols)
    buf.fill_(float("nan"))
    buf[:rows].copy_(cb.to_device(M))
    return buf[:rows]


@pytest.mark.parametrize("seed", range(60 * SCALE))
def test_prod_random_case(cb, seed):
    rng = np.random.default_rng(9000 + seed)
    rf = int(rng.choice([1, 1, 1, 2, 3, 4, 8]))
    h = int(rng.integers(1, 160)) * rf if rf > 1 else int(rng.integers(1, 1400))
    w = int(rng.integers(1, 1400))
    offs = random_offsets(rng, h, w, rf)
    stride = h + int(rng.choice([0, 0, 3, 4]))
    stride += (4 - stride % 4) % 4 if rng.integers(0, 2) else 0
    A = make_dia(rng, h, w, offs, rf, stride=max(stride, h))
    trans = "t" if rng.integers(0, 2) else "n"
    ncols = int(rng.choice([1, 3, 14, 16, 17, 40, 64, 70]))
    fab = float(rng.choice([1.0, 2.0, -0.5]))
    fc = float(rng.choice([0.0, 0.0, 1.0, 1.3]))
    rows_b, rows_c = (h, w) if trans == "t" else (w, h)
    B = F(rng.standard_normal((rows_b, ncols)))
    C0 = F(rng.standard_normal((rows_c, ncols)))
    if fc == 0.0:
        C0[:] = np.nan
    want = C0.copy(order="F")
    ho.prod(want, A, B, trans, fab, fc)
    Cd = device_matrix(cb, rng, C0, bool(rng.integers(0, 2)))
    cb.prod(Cd, to_dev_dia(A), device_matrix(cb, rng, B, bool(rng.integers(0, 2))), trans, "n", fab, fc, cb.MODE_EXACT)
    assert_bits_equal(cb.to_host(Cd), want, "seed %d: prod %s h=%d w=%d rf=%d nd=%d ncols=%d" %
                      (seed, trans, h, w, rf, offs.size, ncols))


@pytest.mark.parametrize("seed", range(30 * SCALE))
def test_dd2dia_random_case(cb, seed):
    rng = np.random.default_rng(9500 + seed)
    rf = int(rng.choice([1, 1, 2, 4]))
    h = int(rng.integers(1, 200)) * rf if rf > 1 else int(rng.integers(1, 1200))
    w = int(rng.integers(1, 1200))
    offs = random_offsets(rng, h, w, rf)
    ncols = int(rng.choice([1, 8, 31, 32, 33, 72, 130]))
    fab, fc = float(rng.choice([1.0, 0.01, -1.0 / 64])), float(rng.choice([0.0, 0.9, 1.0]))
    C = make_dia(rng, h, w, offs, rf, stride=h + (4 - h % 4) % 4)
    X, Y = F(rng.uniform(0, 1, (h, ncols))), F(rng.uniform(0, 1, (w, ncols)))
    want = ho.DiaHost(h, w, C.offsets, C.stride, rf, C.vals.copy())
    m = C.valid_mask().reshape(-1)
    if fc == 0:
        C.vals[m] = np.nan
    ho.densedense_to_dia(want, X, Y, fab, fc, nthreads=4)
    D = to_dev_dia(C)
    pad = bool(rng.integers(0, 2))
    cb.densedense_to_dia(D, None, device_matrix(cb, rng, X, pad), device_matrix(cb, rng, Y, pad), fab, fc)
    got = D.vec.cpu().numpy()
    assert_bits_equal(got[~m], C.vals[~m], "seed %d: cells outside the diagonals' ranges must be untouched" % seed)
    tol = 1e-4 * np.sqrt(max(ncols, 128) / 128.0)
    np.testing.assert_allclose(got[m], want.vals[m], rtol=tol, atol=tol * 1e-3 * max(1.0, abs(fab) * ncols))


@pytest.mark.parametrize("seed", range(6 * SCALE))
def test_prod_random_large_case(cb, seed):
    """Tall matrices with aligned operands: the streaming kernels (at most 16 diagonals on tens of thousands of
    rows), the tiled kernel over many row tiles and the run-walking kernel over many blocks."""
    rng = np.random.default_rng(9800 + seed)
    h = int(rng.integers(8200, 17000)) * 4
    w = h + 4 * int(rng.integers(-500, 500))
    kind = int(rng.integers(0, 3))
    if kind == 0:                                             # narrow band
        nd = int(rng.integers(1, 17)); lo = int(rng.integers(-40, 40)); offs = np.arange(lo, lo + nd)
        ncols = int(rng.choice([1, 5, 32, 40]))
    elif kind == 1:                                           # wide band, many columns
        nd = int(rng.integers(24, 150)); lo = int(rng.integers(-100, 20)); offs = np.arange(lo, lo + nd)
        ncols = int(rng.choice([64, 100, 130]))
    else:                                                     # convolution pattern
        px, fs = int(rng.choice([64, 100, 128])), int(rng.choice([5, 8, 11]))
        offs = np.array([i * px + j for i in range(fs) for j in range(fs)]) - (px + 1) * (fs // 2)
        ncols = int(rng.choice([3, 14, 20]))
    offs = offs.astype(np.int32)
    A = make_dia(rng, h, w, offs, 1, stride=h)
    trans = "t" if rng.integers(0, 2) else "n"
    fab, fc = float(rng.choice([1.0, 2.0])), float(rng.choice([0.0, 1.3]))
    rows_b, rows_c = (h, w) if trans == "t" else (w, h)
    B = F(rng.standard_normal((rows_b, ncols)))
    C0 = F(rng.standard_normal((rows_c, ncols)))
    want = C0.copy(order="F")
    ho.prod(want, A, B, trans, fab, fc, 8)
    Cd = cb.to_device(C0)
    cb.prod(Cd, to_dev_dia(A), cb.to_device(B), trans, "n", fab, fc, cb.MODE_EXACT)
    assert_bits_equal(cb.to_host(Cd), want, "seed %d: prod %s h=%d w=%d nd=%d ncols=%d" %
                      (seed, trans, h, w, offs.size, ncols))


# ---- wider shapes: several row tiles, window segments and waves of blocks per launch ---------------------

def scattered_case(rng, max_rows, spans):
    """Scattered diagonals (stored sorted or not) whose numbers lie within ``span`` of one another around a random
    centre: the span decides which staged-window variant, how many window segments and how many tiles per block."""
    h = int(rng.integers(200, max_rows)); w = int(rng.integers(200, max_rows))
    if rng.integers(0, 2):
        w = h
    nd = int(rng.integers(2, 300 if max_rows > 6000 else 200))
    span = min(int(rng.choice(spans)), (h + w) // 2 - 4)
    c = int(rng.integers(-h + 1 + span // 2, w - 1 - span // 2))
    lo, hi = max(-h + 1, c - span // 2), min(w - 1, c + span // 2)
    nd = min(nd, hi - lo + 1)
    return h, w, rng.choice(np.arange(lo, hi + 1), nd, replace=False).astype(np.int32), span


PROD_SPANS = [64, 300, 900, 1540, 1600, 1650, 2000, 3800, 4560, 4600, 7000]


def wide_prod_case(cb, seed, spans=PROD_SPANS):
    rng = np.random.default_rng(seed)
    h, w, offs, span = scattered_case(rng, 9000, spans)
    if rng.integers(0, 2):
        offs = np.sort(offs)
    stride = h + (4 - h % 4) % 4 if rng.integers(0, 4) else h
    A = make_dia(rng, h, w, offs, 1, stride=stride)
    trans = "t" if rng.integers(0, 2) else "n"
    ncols = int(rng.choice([32, 33, 40, 64, 100, 128, 200]))
    fab = float(rng.choice([1.0, 2.0, -0.5])); fc = float(rng.choice([0.0, 1.0, 1.3]))
    rows_b, rows_c = (h, w) if trans == "t" else (w, h)
    B = F(rng.standard_normal((rows_b, ncols))); C0 = F(rng.standard_normal((rows_c, ncols)))
    if fc == 0.0:
        C0[:] = np.nan
    want = C0.copy(order="F")
    ho.prod(want, A, B, trans, fab, fc, nthreads=8)
    Cd, D = device_matrix(cb, rng, C0, True), to_dev_dia(A)
    cb.prod(Cd, D, device_matrix(cb, rng, B, True), trans, "n", fab, fc, cb.MODE_EXACT)
    assert cb.plan_status(D) == 0
    assert_bits_equal(cb.to_host(Cd), want, "seed %d: prod %s h=%d w=%d nd=%d span=%d ncols=%d" %
                      (seed, trans, h, w, offs.size, span, ncols))


@pytest.mark.parametrize("seed", range(40 * SCALE))
def test_prod_random_scattered_wide_case(cb, seed):
    """Scattered diagonals on matrices of up to 9000 rows times 32-200 aligned batch columns: the staged-window
    kernels with one to five window segments and one to eight row tiles per block, and what the dispatcher picks
    where they do not apply."""
    wide_prod_case(cb, 71000 + seed)


def test_prod_scattered_window_whose_last_segment_is_short(cb):
    """99 unsorted diagonals spanning 1556 on a 1669 x 1669 matrix, transposed: a window of 2071 rows in the
    2176-row variant, whose third segment of 1024 has 23 rows (a copy of the whole segment runs on into the next
    batch column's rows and, from the last column, into the coefficient ring)."""
    wide_prod_case(cb, 70035, [64, 300, 900, 2000, 3800, 7000])


def dd2dia_against_oracle(cb, rng, C, X, Y, fab, fc, pad, what):
    """The sampled product on the device against the host loop: cells outside the diagonals' ranges bit-unchanged,
    the others within the gradient tolerance of the two addends' magnitudes."""
    ncols = X.shape[1]
    want = ho.DiaHost(C.h, C.w, C.offsets, C.stride, C.rf, C.vals.copy())
    m = C.valid_mask().reshape(-1)
    if fc == 0:
        C.vals[m] = np.nan
    ho.densedense_to_dia(want, X, Y, fab, fc, nthreads=8)
    D = to_dev_dia(C)
    cb.densedense_to_dia(D, None, device_matrix(cb, rng, X, pad), device_matrix(cb, rng, Y, pad), fab, fc)
    assert cb.plan_status(D) == 0
    got = D.vec.cpu().numpy()
    assert_bits_equal(got[~m], C.vals[~m], what + ": cells outside the diagonals' ranges must be untouched")
    tol = 1e-4 * np.sqrt(max(ncols, 128) / 128.0)
    bound = np.abs(fc) * np.abs(np.nan_to_num(C.vals[m])) + abs(fab) * ncols      # X, Y in [0, 1)
    err = np.abs(got[m] - want.vals[m])
    assert np.all(err <= tol * bound + 1e-7), what + ": largest error %g of its bound" % float(
        (err / (tol * bound + 1e-7)).max())


@pytest.mark.parametrize("seed", range(30 * SCALE))
def test_dd2dia_random_wide_case(cb, seed):
    """Scattered diagonals on matrices of up to 6000 rows (the windowed kernel: several groups of diagonals per tile,
    groups that leave the matrix) and steep bands with row factors 2-32 (the tiled kernel where the band fills its
    tiles, the windowed one elsewhere), 32-300 batch columns."""
    rng = np.random.default_rng(81000 + seed)
    kind = int(rng.integers(0, 2))
    if kind == 0:
        rf = 1
        h = int(rng.integers(200, 6000)); w = int(rng.integers(200, 6000))
        nd = int(rng.integers(2, 200)); span = min(int(rng.choice([64, 300, 900, 2000])), (h + w) // 2 - 4)
        c = int(rng.integers(-h + 1 + span // 2, w - 1 - span // 2))
        lo, hi = max(-h + 1, c - span // 2), min(w - 1, c + span // 2)
        nd = min(nd, hi - lo + 1)
        offs = rng.choice(np.arange(lo, hi + 1), nd, replace=False).astype(np.int32)
    else:
        rf = int(rng.choice([2, 4, 8, 16, 32]))
        w = int(rng.integers(100, 2000)); h = rf * int(rng.integers(max(1, w // 2), w + w // 2))
        nd = int(rng.integers(8, 200))
        lo_min, hi_max = -(h // rf) + 1, w - 1
        nd = min(nd, hi_max - lo_min + 1)
        lo = int(rng.integers(lo_min, hi_max - nd + 2))
        offs = np.arange(lo, lo + nd, dtype=np.int32)
    ncols = int(rng.choice([32, 64, 72, 128, 256, 300]))
    fab, fc = float(rng.choice([1.0, 0.01, -1.0 / 64])), float(rng.choice([0.0, 0.9, 1.0]))
    C = make_dia(rng, h, w, offs, rf, stride=h + (4 - h % 4) % 4)
    X, Y = F(rng.uniform(0, 1, (h, ncols))), F(rng.uniform(0, 1, (w, ncols)))
    dd2dia_against_oracle(cb, rng, C, X, Y, fab, fc, True, "seed %d: kind=%d rf=%d h=%d w=%d nd=%d ncols=%d" %
                          (seed, kind, rf, h, w, offs.size, ncols))


def regular_pattern(rng, budget):
    """Bands for the tiled kernels, steep bands, convolution patterns, narrow bands on tall matrices and bands times
    few columns, at sizes of several tiles and waves; the batch is halved until the host loop's work fits ``budget``."""
    kind = int(rng.integers(0, 5))
    rf = 1
    if kind == 0:
        h = int(rng.integers(100, 6000)); w = int(rng.integers(100, 6000))
        nd = int(rng.integers(17, 700)); ncols = int(rng.choice([96, 128, 130, 256, 300, 512, 700, 1024]))
    elif kind == 1:
        rf = int(rng.choice([2, 4, 8]))
        w = int(rng.integers(64, 1500)); h = rf * int(rng.integers(max(1, w // 2), w * 2))
        nd = int(rng.integers(8, 300)); ncols = int(rng.choice([64, 200, 256, 512, 1000, 1024, 1100]))
    elif kind == 2:
        h = int(rng.integers(1000, 20000)); w = int(rng.integers(1000, 20000))
        nd = 0; ncols = int(rng.choice([1, 8, 14, 16, 32, 64, 100]))
    elif kind == 3:
        h = int(rng.integers(20000, 300000)); w = h + int(rng.integers(-100, 100))
        nd = int(rng.integers(1, 17)); ncols = int(rng.choice([1, 4, 16, 32, 33]))
    else:
        h = int(rng.integers(1000, 30000)); w = int(rng.integers(1000, 30000))
        nd = int(rng.integers(17, 200)); ncols = int(rng.choice([1, 8, 16, 40, 64, 95]))
    lo_min, hi_max = -((h + rf - 1) // rf) + 1, w - 1
    if kind == 2:
        runs, fs, step = int(rng.integers(2, 12)), int(rng.integers(3, 17)), int(rng.integers(17, 900))
        lo = int(rng.integers(lo_min, max(lo_min + 1, hi_max - runs * step - fs)))
        offs = np.concatenate([lo + r * step + np.arange(fs) for r in range(runs)])
        offs = offs[(offs >= lo_min) & (offs <= hi_max)]
        if offs.size == 0:
            offs = np.array([0])
        if rng.integers(0, 3) == 0:
            offs = np.concatenate([offs, offs])
    else:
        nd = min(nd, hi_max - lo_min + 1)
        mode = int(rng.integers(0, 3))
        if mode == 0:
            lo = int(rng.integers(lo_min, hi_max - nd + 2))
        elif mode == 1:
            lo = -nd // 2                       # may reach past the last column: diagonals that hold no cell
        else:
            lo = int(np.clip(int(rng.integers(-300, 300)), lo_min, hi_max - nd + 1))
        offs = np.arange(lo, lo + nd)
    offs = offs.astype(np.int32)
    while h * offs.size * ncols > budget and ncols > 1:
        ncols = max(1, ncols // 2)
    return kind, h, w, rf, offs, ncols


@pytest.mark.parametrize("seed", range(40 * SCALE))
def test_prod_random_regular_wide_case(cb, seed):
    rng = np.random.default_rng(72000 + seed)
    kind, h, w, rf, offs, ncols = regular_pattern(rng, 6e8)
    al = bool(rng.integers(0, 4))
    stride = h + (4 - h % 4) % 4 if al else h + int(rng.choice([0, 1, 3]))
    A = make_dia(rng, h, w, offs, rf, stride=stride)
    trans = "t" if rng.integers(0, 2) else "n"
    fab = float(rng.choice([1.0, 2.0, -0.5])); fc = float(rng.choice([0.0, 1.0, 1.3]))
    rows_b, rows_c = (h, w) if trans == "t" else (w, h)
    B = F(rng.standard_normal((rows_b, ncols))); C0 = F(rng.standard_normal((rows_c, ncols)))
    if fc == 0.0:
        C0[:] = np.nan
    want = C0.copy(order="F")
    ho.prod(want, A, B, trans, fab, fc, nthreads=8)
    Cd, D = device_matrix(cb, rng, C0, al), to_dev_dia(A)
    cb.prod(Cd, D, device_matrix(cb, rng, B, al), trans, "n", fab, fc, cb.MODE_EXACT)
    assert cb.plan_status(D) == 0
    assert_bits_equal(cb.to_host(Cd), want, "seed %d: kind=%d prod %s h=%d w=%d rf=%d nd=%d lo=%d ncols=%d al=%d" %
                      (seed, kind, trans, h, w, rf, offs.size, offs[0], ncols, al))


@pytest.mark.parametrize("seed", range(30 * SCALE))
def test_dd2dia_random_regular_wide_case(cb, seed):
    rng = np.random.default_rng(82000 + seed)
    kind, h, w, rf, offs, ncols = regular_pattern(rng, 3e8)
    ncols = max(ncols, 2)
    fab, fc = float(rng.choice([1.0, 0.01, -1.0 / 64])), float(rng.choice([0.0, 0.9, 1.0]))
    al = bool(rng.integers(0, 4))
    C = make_dia(rng, h, w, offs, rf, stride=h + (4 - h % 4) % 4 if al else h)
    X, Y = F(rng.uniform(0, 1, (h, ncols))), F(rng.uniform(0, 1, (w, ncols)))
    dd2dia_against_oracle(cb, rng, C, X, Y, fab, fc, al, "seed %d: kind=%d rf=%d h=%d w=%d nd=%d lo=%d ncols=%d al=%d" %
                          (seed, kind, rf, h, w, offs.size, offs[0], ncols, al))
