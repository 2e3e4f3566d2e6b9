"""BASELINE-size checks through size-independent properties (the oracle is too slow for whole outputs
at these sizes): bit-exact comparison with the oracle on a slice of batch columns, the adjoint
identity that ties prod 'n' to prod 't', the trace identity that ties densedense_to_dia to prod,
linearity, checksum-of-checksums for the reductions, and untouched padding cells.

Shapes: config 3 in full (16384 x 16384, 512 diagonals, batch 1024), the per-GPU shard of config 4
at 8 GPUs (65536 x 65536, 1024 diagonals, batch 1024) and config 4 with the whole batch of 8192 on one GPU
(the benchmark's one-GPU shape: 64 column tiles of the banded product, oracle slices on columns that fall
into different tiles); config 1 in full (16384 x 4096, rf 4, 256
diagonals, batch 512); config 0 and 2 run in full in test_gpu_parity.py."""
import numpy as np
import pytest

from oracle import host_oracle as ho
from tests.helpers import assert_bits_equal

pytestmark = pytest.mark.gpu


def dot64(a, b):
    return float((a.double() * b.double()).sum().item())


def band_problem(cb, n, nd, nb, seed):
    import torch
    g = torch.Generator(device="cuda")
    g.manual_seed(seed)
    offs = np.arange(-nd // 2, nd // 2, dtype=np.int32)
    W = cb.dev_dia_matrix_f(n, n, offs, n, 1)
    W.vec.normal_(0.0, 0.01, generator=g)
    X = cb.colmajor_empty(n, nb)
    X.t().copy_(torch.rand((nb, n), device="cuda", generator=g) * 2 - 1)
    Y = cb.colmajor_empty(n, nb)
    Y.t().copy_(torch.rand((nb, n), device="cuda", generator=g) * 2 - 1)
    return W, offs, X, Y


@pytest.mark.parametrize("n,nd,nb", [(16384, 512, 1024), (65536, 1024, 1024), (65536, 1024, 8192)])
def test_band_full_size_properties(n, nd, nb):
    import torch
    import cuv_b200 as cb
    W, offs, X, Y = band_problem(cb, n, nd, nb, 4000 + nd)
    mask = torch.from_numpy(ho.DiaHost(n, n, offs, n, 1).valid_mask().reshape(-1)).cuda()
    W.vec[~mask] = float("nan")                                   # padding must never be read
    WX, WtY = cb.colmajor_empty(n, nb), cb.colmajor_empty(n, nb)
    cb.prod(WX, W, X, "n", "n", 1.0, 0.0, cb.MODE_EXACT)
    cb.prod(WtY, W, Y, "t", "n", 1.0, 0.0, cb.MODE_EXACT)
    assert torch.isfinite(WX).all() and torch.isfinite(WtY).all()
    # 1. a slice of batch columns against the oracle, bit for bit (both directions)
    Wh = ho.DiaHost(n, n, offs, n, 1, W.vec.cpu().numpy())
    cols = [0, 1, nb // 2, nb - 1] if nb <= 1024 else [0, 127, 128, nb // 2 - 1, nb - 1]
    sl = lambda t: np.asfortranarray(t[:, cols].cpu().numpy())          # the slice is taken on the device
    Xs, Ys = sl(X), sl(Y)
    want = np.zeros((n, len(cols)), dtype=np.float32, order="F")
    ho.prod(want, Wh, Xs, "n", nthreads=8)
    assert_bits_equal(sl(WX), want, "prod 'n' slice at full size")
    ho.prod(want, Wh, Ys, "t", nthreads=8)
    assert_bits_equal(sl(WtY), want, "prod 't' slice at full size")
    # 2. adjoint identity <W X, Y> == <X, W^T Y>
    # (the products have random signs, so the tolerance is relative to the sum of |terms|: fp32 rounding of
    # each of the n*nb outputs, about 6e-8 of its size, is all that separates the two sides)
    lhs, rhs = dot64(WX, Y), dot64(X, WtY)
    scale = dot64(WX.abs(), Y.abs())
    assert abs(lhs - rhs) <= 1e-7 * scale
    # 3. trace identity: sum over stored cells of W * dd2dia(Y, X) == <Y, W X>   (G = Y X^T on the band)
    G = cb.dev_dia_matrix_f(n, n, offs, n, 1)
    G.vec.fill_(7.0)
    cb.densedense_to_dia(G, None, Y, X, 1.0, 0.0)
    assert bool((G.vec[~mask] == 7.0).all()), "cells outside the diagonals' ranges were written"
    tr = float((G.vec[mask].double() * W.vec[mask].double()).sum().item())
    assert abs(tr - lhs) <= 1e-6 * scale
    # ... and a few diagonals of G against the oracle on all batch columns
    some = [0, nd // 2, nd - 1]
    sub = ho.DiaHost(n, n, offs[some], n, 1)
    ho.densedense_to_dia(sub, cb.to_host(Y), cb.to_host(X), 1.0, 0.0, nthreads=8)
    got = G.vec.cpu().numpy().reshape(nd, n)[some]
    m = sub.valid_mask()
    tol = 1e-4 * np.sqrt(nb / 128.0)
    np.testing.assert_allclose(got[m], sub.vals.reshape(len(some), n)[m], rtol=tol, atol=tol)
    # 4. factC: C <- 0.5*C + 1*W X applied to C = W X gives 1.5 * W X exactly (scaling by 0.5 and the sum are exact)
    C2 = WX.clone()
    cb.prod(C2, W, X, "n", "n", 1.0, 0.5, cb.MODE_EXACT)
    refh = sl(WX).copy(order="F")
    ho.prod(refh, Wh, Xs, "n", 1.0, 0.5, nthreads=8)
    assert_bits_equal(sl(C2), refh, "factC path at full size")
    del C2
    # 5. reductions: checksum of checksums
    v = torch.empty(n, device="cuda")
    cb.reduce_to_col(v, WX)
    total = float(WX.double().sum().item())
    assert abs(float(v.double().sum().item()) - total) <= 1e-6 * float(WX.double().abs().sum().item())
    r = torch.empty(nb, device="cuda")
    cb.reduce_to_row(r, WX)
    assert abs(float(r.double().sum().item()) - total) <= 1e-6 * float(WX.double().abs().sum().item())
    # 6. FAST arithmetic stays within one rounding per term of EXACT
    WXf = cb.colmajor_empty(n, nb)
    cb.prod(WXf, W, X, "n", "n", 1.0, 0.0, cb.MODE_FAST)
    WXf.sub_(WX)
    assert float(WXf.abs().max().item()) <= 1e-5 * float(WX.abs().max().item())
    assert cb.plan_status(W) == 0 and cb.plan_status(G) == 0


def test_config1_full_size_properties():
    """Transposed product with row factor 4 (config 1): oracle slice, adjoint identity with 'n', factC."""
    import torch
    import cuv_b200 as cb
    h, w, nd, rf, nb = 16384, 4096, 256, 4, 512
    g = torch.Generator(device="cuda")
    g.manual_seed(1001)
    offs = np.arange(-128, 128, dtype=np.int32)
    A = cb.dev_dia_matrix_f(h, w, offs, h, rf)
    A.vec.uniform_(-1, 1, generator=g)
    mask = torch.from_numpy(ho.DiaHost(h, w, offs, h, rf).valid_mask().reshape(-1)).cuda()
    A.vec[~mask] = float("nan")
    B = cb.colmajor_empty(h, nb); B.t().copy_(torch.rand((nb, h), device="cuda", generator=g) * 2 - 1)
    C0 = cb.colmajor_empty(w, nb); C0.t().copy_(torch.rand((nb, w), device="cuda", generator=g) * 2 - 1)
    C = C0.clone()
    cb.prod(C, A, B, "t", "n", 1.0, 0.5, cb.MODE_EXACT)
    Ah = ho.DiaHost(h, w, offs, h, rf, A.vec.cpu().numpy())
    cols = [0, 255, 511]
    want = np.asfortranarray(cb.to_host(C0)[:, cols]).copy(order="F")
    ho.prod(want, Ah, np.asfortranarray(cb.to_host(B)[:, cols]), "t", 1.0, 0.5, nthreads=8)
    assert_bits_equal(np.asfortranarray(cb.to_host(C)[:, cols]), want, "config 1 slice")
    # adjoint: <A^T B, Y> == <B, A Y>
    Y = cb.colmajor_empty(w, nb); Y.t().copy_(torch.rand((nb, w), device="cuda", generator=g))
    AtB, AY = cb.colmajor_empty(w, nb), cb.colmajor_empty(h, nb)
    cb.prod(AtB, A, B, "t")
    cb.prod(AY, A, Y, "n")
    lhs, rhs = dot64(AtB, Y), dot64(B, AY)
    assert abs(lhs - rhs) <= 1e-7 * dot64(AtB.abs(), Y.abs())
