"""The CPU oracle against the known-answer fixtures of CUV's own tests (tests/golden/make_golden.py)
and against float64 dense computations for the cases the reference never tests."""
import numpy as np
import pytest

from oracle import host_oracle as ho


def F(a):
    return np.asfortranarray(a, dtype=np.float32)


def test_dia_to_dense_matches_reference_fixture(golden):
    g = golden
    A = ho.DiaHost(int(g["diamat_h"]), int(g["diamat_w"]), g["diamat_offsets"], int(g["diamat_stride"]), 1,
                   g["diamat_vals"])
    assert np.array_equal(A.to_dense(), g["diamat_dense"])        # src/tests/dia_mat.cpp:111-119
    A = ho.DiaHost(int(g["spmv_h"]), int(g["spmv_w"]), g["spmv_offsets"], int(g["spmv_stride"]), 1, g["spmv_vals"])
    assert np.array_equal(A.to_dense(), g["spmv_dense"])
    for i in range(A.h):
        for j in range(A.w):
            c = A.cell_index(i, j)
            assert (c < 0) == (abs(j - i) > 3)
            if c >= 0:
                assert A.vals[c] == g["spmv_dense"][i, j]


def _spmv_fixture(g):
    A = ho.DiaHost(int(g["spmv_h"]), int(g["spmv_w"]), g["spmv_offsets"], int(g["spmv_stride"]),
                   int(g["spmv_rf"]), g["spmv_vals"])
    return A, F(g["spmv_B"]), F(g["spmv_C"])


def test_prod_trans_defaults_matches_reference_fixture(golden):
    A, B, C = _spmv_fixture(golden)                                  # src/tests/spmv.cpp:103-115
    out = F(np.full_like(B, np.nan))                                 # factC == 0: old contents must not matter
    ho.prod(out, A, C, "t")
    assert np.array_equal(out.astype(np.float64), golden["spmv_expect_t_1_0"])   # integers < 2^24: exact


def test_prod_n_2_13_matches_reference_fixture(golden):
    A, B, C = _spmv_fixture(golden)                                  # src/tests/spmv.cpp:116-136
    ho.prod(C, A, B, "n", 2.0, 1.3)
    np.testing.assert_allclose(C, golden["spmv_expect_n_2_13"], rtol=1e-6)


def test_prod_t_2_13_matches_reference_fixture(golden):
    A, B, C = _spmv_fixture(golden)                                  # src/tests/spmv.cpp:137-143
    ho.prod(B, A, C, "t", 2.0, 1.3)
    np.testing.assert_allclose(B, golden["spmv_expect_t_2_13"], rtol=1e-6)


@pytest.mark.parametrize("literal", [False, True])
def test_dd2dia_matches_reference_fixture(golden, literal):
    g = golden                                                        # src/tests/densedense_to_dia.cpp:139-197
    C = ho.DiaHost(int(g["dd2dia_h"]), int(g["dd2dia_w"]), g["dd2dia_offsets"], int(g["dd2dia_stride"]),
                   int(g["dd2dia_rf"]))
    ho.densedense_to_dia(C, F(g["dd2dia_A"]), F(g["dd2dia_B"]), literal_host=literal)
    assert np.array_equal(C.vals.astype(np.float64), g["dd2dia_expect"])          # exact integers
    assert np.array_equal(C.valid_mask().reshape(-1), g["dd2dia_mask"])


def test_dd2dia_padding_untouched_and_factors():
    rng = np.random.default_rng(5)
    h, w, rf, nb = 24, 11, 2, 9
    offs = np.array([3, -2, 0, 7, -11], dtype=np.int32)
    C = ho.DiaHost(h, w, offs, 32, rf, rng.standard_normal(5 * 32).astype(np.float32))
    old = C.vals.copy()
    X, H = F(rng.standard_normal((h, nb))), F(rng.standard_normal((w, nb)))
    ho.densedense_to_dia(C, X, H, 0.25, 0.5)
    m = C.valid_mask().reshape(-1)
    assert np.array_equal(C.vals[~m], old[~m])
    dense = X.astype(np.float64) @ H.astype(np.float64).T
    for s, k in enumerate(offs.tolist()):
        for i in range(h):
            j = i // rf + k
            if 0 <= j < w:
                assert m[s * 32 + i]
                np.testing.assert_allclose(C.vals[s * 32 + i], 0.5 * old[s * 32 + i] + 0.25 * dense[i, j],
                                           rtol=2e-5, atol=2e-6)
            else:
                assert not m[s * 32 + i]


@pytest.mark.parametrize("rf", [1, 2, 4])
@pytest.mark.parametrize("trans", ["n", "t"])
def test_prod_row_fact_vs_float64_dense(rf, trans):
    """Not pinned by any reference test (prod with row_fact > 1 is host-only code the reference never
    exercises): checked against a float64 dense product of the dia->dense conversion."""
    rng = np.random.default_rng(10 * rf + (trans == "t"))
    w, nb = 13, 5
    h = rf * 10
    offs = np.array([-9, 4, 0, -1, 12, 2], dtype=np.int32)          # user order, unsorted
    A = ho.DiaHost(h, w, offs, h + 3, rf, rng.standard_normal(6 * (h + 3)).astype(np.float32))
    A.vals[~A.valid_mask().reshape(-1)] = np.nan                     # padding must never be read
    D = A.to_dense().astype(np.float64)
    if trans == "n":
        B, C = F(rng.standard_normal((w, nb))), F(rng.standard_normal((h, nb)))
        ref = 0.5 * C.astype(np.float64) + 1.5 * (D @ B)
    else:
        B, C = F(rng.standard_normal((h, nb))), F(rng.standard_normal((w, nb)))
        ref = 0.5 * C.astype(np.float64) + 1.5 * (D.T @ B)
    ho.prod(C, A, B, trans, 1.5, 0.5)
    np.testing.assert_allclose(C, ref, rtol=1e-5, atol=1e-5)


def test_prod_threads_bit_identical():
    rng = np.random.default_rng(3)
    h = w = 257
    offs = np.sort(rng.choice(np.arange(-200, 201), 17, replace=False)).astype(np.int32)
    A = ho.DiaHost(h, w, offs, h, 1, rng.uniform(-1, 1, 17 * h).astype(np.float32))
    B = F(rng.uniform(-1, 1, (w, 33)))
    C1, C2 = F(np.zeros((h, 33))), F(np.zeros((h, 33)))
    ho.prod(C1, A, B, nthreads=1)
    ho.prod(C2, A, B, nthreads=5)
    assert np.array_equal(C1, C2)


NAMES = {ho.RF_ADD: "add", ho.RF_MAX: "max", ho.RF_MIN: "min", ho.RF_ARGMAX: "argmax", ho.RF_ARGMIN: "argmin",
         ho.RF_LOGADDEXP: "logaddexp", ho.RF_ADD_SQUARED: "addsq"}


@pytest.mark.parametrize("rf", sorted(NAMES))
@pytest.mark.parametrize("over_strided", [True, False])
def test_reduce_matches_reference_fixture(golden, rf, over_strided):
    src = F(golden["reduce_src"])                                    # src/tests/matrix_op.cpp:858-924
    dst = np.full(270, np.nan, dtype=np.float32)
    ho.reduce(dst, src, over_strided, rf, nthreads=3)
    want = golden["reduce_%s_over_%s" % (NAMES[rf], "cols" if over_strided else "rows")]
    if rf in (ho.RF_ARGMAX, ho.RF_ARGMIN):
        assert np.array_equal(dst.astype(np.int64), want)
    else:
        np.testing.assert_allclose(dst, want, rtol=1e-5)


def test_reduce_factors_mean_mult():
    rng = np.random.default_rng(9)
    src = F(rng.uniform(0.5, 1.5, (37, 21)))
    old = rng.standard_normal(37).astype(np.float32)
    dst = old.copy()
    ho.reduce_to_col(dst, src, ho.RF_ADD, 0.25, 0.5)
    np.testing.assert_allclose(dst, 0.5 * old + 0.25 * src.astype(np.float64).sum(1), rtol=1e-5)
    dst = np.zeros(21, dtype=np.float32)
    ho.reduce_to_row(dst, src, ho.RF_MEAN)
    np.testing.assert_allclose(dst, src.astype(np.float64).mean(0), rtol=1e-5)
    ho.reduce_to_row(dst, src, ho.RF_MULT)
    np.testing.assert_allclose(dst, src.astype(np.float64).prod(0), rtol=1e-4)
    ho.reduce_to_row(dst, src, ho.RF_ADDEXP)
    np.testing.assert_allclose(dst, np.exp(src.astype(np.float64)).sum(0), rtol=1e-4)
    with pytest.raises(RuntimeError):
        ho.reduce_to_row(dst, src, ho.RF_MEAN, 2.0, 0.0)


def test_bias_sigmoid_sample():
    rng = np.random.default_rng(2)
    a = F(rng.standard_normal((19, 7)))
    b = rng.standard_normal(19).astype(np.float32)
    u = F(rng.uniform(0, 1, (19, 7)))
    p = 1.0 / (1.0 + np.exp(-(a.astype(np.float64) + b[:, None])))
    s = ho.bias_sigmoid_sample(a, b, u)
    np.testing.assert_allclose(a, p, rtol=1e-6)
    assert np.array_equal(s, (a > u).astype(np.float32))


def test_learn_step_weight_decay_oracle():
    """The update step's restatement against the formula spelled out in numpy float32, and the reference's own
    test of it (src/tests/optimize.cpp:59-87,89-121): 1000 steps on f(W) = 2 (W - optimum)^2 reach the optimum."""
    rng = np.random.default_rng(7)
    w, g = rng.standard_normal(1001).astype(np.float32), rng.standard_normal(1001).astype(np.float32)
    lr, decay = np.float32(0.1), np.float32(0.05)
    want = (-lr) * g + (np.float32(1) - lr * decay) * w
    got = ho.learn_step_weight_decay(w.copy(), g, 0.1, 0.05)
    assert np.array_equal(got.view(np.uint32), want.astype(np.float32).view(np.uint32))
    for momentum in (False, True):
        N = 8092
        opt, W = rng.random(N, dtype=np.float32), rng.random(N, dtype=np.float32)
        M = np.zeros(N, dtype=np.float32)
        for it in range(1000):
            dW = W - opt
            if momentum:
                ho.learn_step_weight_decay_momentum(W, M, dW, 0.01, 1.0 - it / 1000.0, 0.0)
            else:
                ho.learn_step_weight_decay(W, dW, 0.01, 0.0)
        np.testing.assert_allclose(W + 1, opt + 1, rtol=1e-4)
    # with a decay the reference's host loop and device kernel differ in one sign; both are restated
    w1, w2, m1, m2 = w.copy(), w.copy(), np.zeros_like(w), np.zeros_like(w)
    ho.learn_step_weight_decay_momentum(w1, m1, g, 0.1, 0.9, 0.05, device_formula=True)
    ho.learn_step_weight_decay_momentum(w2, m2, g, 0.1, 0.9, 0.05, device_formula=False)
    assert np.array_equal(m1, -lr * (g + decay * w)) and np.array_equal(m2, -lr * (g - decay * w))


def test_typed_reductions_follow_the_host_loop():
    """Known answers for the reductions between other element types, worked out by hand from CUV's host loop
    (matrix_ops/matrix_ops_reduce.cu:217-292): the running value has the SOURCE type, the fold computes in the
    DESTINATION type, factors are converted to the source type."""
    import numpy as np
    from oracle import host_oracle as ho
    m8 = np.asfortranarray(np.array([[0, 30, 60, 90], [120, 150, 180, 210], [240, 14, 44, 74]], dtype=np.uint8))
    d = np.zeros(3, dtype=np.float32)
    assert ho.reduce_typed(d, m8, True).tolist() == [180.0, 660 % 256, 372 % 256]      # 8-bit running value wraps
    d = np.zeros(3, dtype=np.uint32)
    assert ho.reduce_typed(d, m8, True, ho.RF_MAX).tolist() == [90, 210, 240]
    d = np.zeros(4, dtype=np.uint8)
    assert ho.reduce_typed(d, m8, False, ho.RF_ARGMAX).tolist() == [2, 1, 1, 1]
    d = np.full(4, 7, dtype=np.uint8)
    assert ho.reduce_typed(d, m8, False, ho.RF_ARGMIN).tolist() == [0, 2, 2, 2]
    mf = np.asfortranarray(np.array([[1.7, 2.2, -3.9], [0.5, 100.9, 7.0]], dtype=np.float32))
    d = np.array([10, 20], dtype=np.int32)
    # float -> int: every element is truncated before it is added; factors stay float: 0.5*old + 2*sum, then truncated
    assert ho.reduce_typed(d, mf, True, ho.RF_ADD, 2.0, 0.5).tolist() == [int(0.5 * 10 + 2 * 0), int(0.5 * 20 + 2 * 107)]
    mi = np.asfortranarray(np.array([[3, -4], [5, 6]], dtype=np.int32))
    d = np.array([1.5, 2.5], dtype=np.float32)
    # int -> float: factors are converted to int first (2.9 -> 2, 0.9 -> 0: the old value is dropped)
    assert ho.reduce_typed(d, mi, True, ho.RF_ADD, 2.9, 0.9).tolist() == [-2.0, 22.0]
    assert ho.reduce_typed(np.zeros(2, dtype=np.float32), mi, True, ho.RF_ADD_SQUARED).tolist() == [25.0, 61.0]
    assert ho.reduce_typed(np.zeros(2, dtype=np.float32), mi, False, ho.RF_MEAN).tolist() == [4.0, 1.0]
    with pytest.raises(RuntimeError):
        ho.reduce_typed(np.zeros(2, dtype=np.int32), mi, True)          # int -> int is not instantiated by CUV


def test_avg_diagonals_fixture():
    """src/tests/dia_mat.cpp:134-142 (the call is commented out there): each diagonal's mean over its cells inside
    the matrix; a 4 x 3 matrix whose diagonals hold 1..n along their valid range."""
    import numpy as np
    from oracle import host_oracle as ho
    A = ho.DiaHost(4, 3, np.array([0, 1, -2], dtype=np.int32), 4, 1)
    A.vals[:] = np.nan
    A.vals[0:3] = [1, 2, 3]            # diagonal 0: cells (0,0) (1,1) (2,2)
    A.vals[4:6] = [4, 6]               # diagonal +1: cells (0,1) (1,2)
    A.vals[10:12] = [10, 20]           # diagonal -2: cells (2,0) (3,1), stored at rows 2, 3
    out = np.zeros(3, dtype=np.float32)
    assert ho.avg_diagonals(out, A).tolist() == [2.0, 5.0, 15.0]


def test_philox_known_answers():
    """The generator behind the product path's device-drawn uniform numbers, against the known-answer vectors its
    authors publish for Philox4x32 with 10 rounds (counter, key -> output), and the mapping to [0, 1)."""
    kat = [
        ((0, 0, 0, 0), (0, 0), (0x6627e8d5, 0xe169c58d, 0xbc57ac4c, 0x9b00dbd8)),
        ((0xffffffff,) * 4, (0xffffffff,) * 2, (0x408f276d, 0x41c83b0e, 0xa20bc7c6, 0x6d5451fd)),
        ((0x243f6a88, 0x85a308d3, 0x13198a2e, 0x03707344), (0xa4093822, 0x299f31d0),
         (0xd16cfe09, 0x94fdcceb, 0x5001e420, 0x24126ea1)),
    ]
    for ctr, key, want in kat:
        assert tuple(int(x) for x in ho.philox4x32_10(ctr, key)) == want
    # element (row, column) of draw `which` in step `step`: word row % 4 of the block with counter
    # (row / 4, column, which, step), as (word >> 8) * 2^-24
    u = ho.uniform(7, 3, seed=0x299f31d0a4093822, step=0x03707344, col0=0x85a308d3 - 1, which=0)
    blk = ho.philox4x32_10((1, 0x85a308d3, 0, 0x03707344), (0xa4093822, 0x299f31d0))
    assert u[4, 1] == np.float32(int(blk[0]) >> 8) * np.float32(2.0 ** -24)
    assert u[6, 1] == np.float32(int(blk[2]) >> 8) * np.float32(2.0 ** -24)
    big = ho.uniform(1000, 40, seed=7, step=1, which=1)
    assert 0.0 <= big.min() and big.max() < 1.0 and abs(big.mean() - 0.5) < 0.01
