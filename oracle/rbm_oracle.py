"""CPU oracle of the sparse-RBM CD-1 step (TEST INFRASTRUCTURE ONLY, like everything in oracle/).

Same call order as examples/rbm/base.py:223-258 of CUV with one Gibbs step and the dense weight
products replaced by their DIA forms; every routine is the host oracle of ``host_oracle``.
"""
import numpy as np

from . import host_oracle as ho


def make_inputs(seed, hid, vis, offsets, nb, p_vis=0.3, w_std=0.01, tie_margin=1e-4, nthreads=8):
    """Seeded inputs of one step: W ~ N(0, w_std) on the stored cells, V0 ~ Bernoulli(p_vis), and
    uniforms U_h, U_v in [0,1).  Uniforms closer than ``tie_margin`` to the probability they are compared
    with are moved away from it, so that sampling is insensitive to last-bit differences between
    the CPU's and the GPU's expf."""
    rng = np.random.Generator(np.random.PCG64(seed))
    offsets = np.asarray(offsets, dtype=np.int32)
    W = ho.DiaHost(hid, vis, offsets, max(hid, vis), 1,
                   (rng.standard_normal(offsets.size * max(hid, vis)) * w_std).astype(np.float32))
    V0 = np.asfortranarray((rng.random((vis, nb), dtype=np.float32) < p_vis).astype(np.float32))
    U_h = np.asfortranarray(rng.random((hid, nb), dtype=np.float32))
    U_v = np.asfortranarray(rng.random((vis, nb), dtype=np.float32))
    b = np.zeros(vis, dtype=np.float32)
    c = np.zeros(hid, dtype=np.float32)

    def away(p, u):
        near = np.abs(p - u) < tie_margin
        u[near] = np.where(p[near] >= 0.5, p[near] - 10 * tie_margin, p[near] + 10 * tie_margin)

    H0p = np.zeros((hid, nb), dtype=np.float32, order="F")
    ho.prod(H0p, W, V0, "n", nthreads=nthreads)
    ho.bias_sigmoid_sample(H0p, c, None, nthreads)
    away(H0p, U_h)
    H0 = np.asfortranarray((H0p > U_h).astype(np.float32))
    V1p = np.zeros((vis, nb), dtype=np.float32, order="F")
    ho.prod(V1p, W, H0, "t", nthreads=nthreads)
    ho.bias_sigmoid_sample(V1p, b, None, nthreads)
    away(V1p, U_v)
    return W, V0, U_h, U_v


def cd1_step(W, V0, U_h, U_v, batch_global=None, b=None, c=None, nthreads=1):
    """Returns dict(H0p, H0, V1p, V1, H1p, G (DiaHost), gc, gb) for the given batch columns."""
    hid, vis, nb = W.h, W.w, V0.shape[1]
    inv = np.float32(1.0 / (batch_global if batch_global else nb))
    b = np.zeros(vis, dtype=np.float32) if b is None else b
    c = np.zeros(hid, dtype=np.float32) if c is None else c
    H0p = np.zeros((hid, nb), dtype=np.float32, order="F")
    ho.prod(H0p, W, V0, "n", nthreads=nthreads)
    H0 = ho.bias_sigmoid_sample(H0p, c, U_h, nthreads)
    V1p = np.zeros((vis, nb), dtype=np.float32, order="F")
    ho.prod(V1p, W, H0, "t", nthreads=nthreads)
    V1 = ho.bias_sigmoid_sample(V1p, b, U_v, nthreads)
    H1p = np.zeros((hid, nb), dtype=np.float32, order="F")
    ho.prod(H1p, W, V1, "n", nthreads=nthreads)
    ho.bias_sigmoid_sample(H1p, c, None, nthreads)
    G = ho.DiaHost(hid, vis, W.offsets, W.stride, W.rf)
    ho.densedense_to_dia(G, H0p, V0, float(inv), 0.0, nthreads=nthreads)
    ho.densedense_to_dia(G, H1p, V1, float(-inv), 1.0, nthreads=nthreads)
    gc, gb = np.zeros(hid, dtype=np.float32), np.zeros(vis, dtype=np.float32)
    ho.reduce_to_col(gc, H0p, ho.RF_ADD, float(inv), 0.0, nthreads)
    ho.reduce_to_col(gc, H1p, ho.RF_ADD, float(-inv), 1.0, nthreads)
    ho.reduce_to_col(gb, V0, ho.RF_ADD, float(inv), 0.0, nthreads)
    ho.reduce_to_col(gb, V1, ho.RF_ADD, float(-inv), 1.0, nthreads)
    return dict(H0p=H0p, H0=H0, V1p=V1p, V1=V1, H1p=H1p, G=G, gc=gc, gb=gb)
