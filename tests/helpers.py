"""Shared input builders for the parity tests: seeded, bit-identical inputs for the oracle and the GPU."""
import numpy as np

from oracle import host_oracle as ho


def F(a):
    return np.asfortranarray(a, dtype=np.float32)


def make_dia(rng, h, w, offsets, rf=1, stride=None, poison=True, dist="uniform", scale=1.0):
    """Host DIA matrix with seeded values; cells no routine may read are NaN when ``poison``."""
    offsets = np.asarray(offsets, dtype=np.int32)
    stride = stride if stride is not None else max(h, w)
    n = offsets.size * stride
    vals = (rng.uniform(-1, 1, n) if dist == "uniform" else rng.standard_normal(n) * scale).astype(np.float32)
    A = ho.DiaHost(h, w, offsets, stride, rf, vals)
    if poison:
        A.vals[~A.valid_mask().reshape(-1)] = np.nan
    return A


def to_dev_dia(A, device="cuda"):
    import cuv_b200 as cb
    D = cb.dev_dia_matrix_f(A.h, A.w, A.offsets, A.stride, A.rf, device=device)
    D.set_vec(A.vals)
    return D


def scattered_offsets(rng, n, lo, hi, sort=True):
    o = rng.choice(np.arange(lo, hi + 1), n, replace=False)
    return (np.sort(o) if sort else o).astype(np.int32)


def assert_bits_equal(got, want, what=""):
    got, want = np.asarray(got), np.asarray(want)
    assert got.shape == want.shape, what
    g, w = got.view(np.uint32), want.view(np.uint32)
    # +0 and -0 compare equal numerically; everything else must match bit for bit (NaNs included)
    bad = (g != w) & ~((got == 0) & (want == 0))
    assert not bad.any(), "%s: %d of %d elements differ, first at %s: got %r want %r" % (
        what, int(bad.sum()), bad.size, np.argwhere(bad)[0], got[tuple(np.argwhere(bad)[0])],
        want[tuple(np.argwhere(bad)[0])])
