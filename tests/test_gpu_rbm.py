"""The sparse-RBM CD-1 step on the GPU against the CPU oracle's step (same seeded inputs)."""
import numpy as np
import pytest

from oracle import host_oracle as ho
from oracle import rbm_oracle
from tests.helpers import assert_bits_equal

pytestmark = pytest.mark.gpu


def run_gpu_step(cb, W, V0, U_h, U_v, batch_global=None, mode=None, fused=True):
    from cuv_b200 import rbm
    Wd = cb.dev_dia_matrix_f(W.h, W.w, W.offsets, W.stride, W.rf).set_vec(W.vals)
    st = rbm.SparseRBMStep(Wd, V0.shape[1], batch_global, cb.MODE_EXACT if mode is None else mode, fused=fused)
    st.step(cb.to_device(V0), cb.to_device(U_h), cb.to_device(U_v))
    return st


@pytest.mark.parametrize("units,nd,nb", [(1024, 32, 96), (2048, 128, 160)])
def test_cd1_step_matches_oracle(units, nd, nb):
    import cuv_b200 as cb
    offs = np.arange(-nd // 2, nd // 2, dtype=np.int32)
    W, V0, U_h, U_v = rbm_oracle.make_inputs(1003, units, units, offs, nb, w_std=0.05)
    ref = rbm_oracle.cd1_step(W, V0, U_h, U_v, nthreads=8)
    st = run_gpu_step(cb, W, V0, U_h, U_v)
    np.testing.assert_allclose(cb.to_host(st.H0p), ref["H0p"], rtol=1e-5)           # activations: rel 1e-5
    assert np.array_equal(cb.to_host(st.H0), ref["H0"])                              # samples identical
    np.testing.assert_allclose(cb.to_host(st.V1p), ref["V1p"], rtol=1e-5)
    assert np.array_equal(cb.to_host(st.V1), ref["V1"])
    np.testing.assert_allclose(cb.to_host(st.H1p), ref["H1p"], rtol=1e-5)
    # gradients are differences of two batch sums: compare against the size of the summands
    tol = 1e-4 * np.sqrt(max(nb, 128) / 128.0)
    m = ref["G"].valid_mask().reshape(-1)
    got = st.G.vec.cpu().numpy()
    scale = np.zeros_like(got)
    pos = ho.DiaHost(W.h, W.w, W.offsets, W.stride, 1)
    ho.densedense_to_dia(pos, ref["H0p"], V0, 1.0 / nb, 0.0, nthreads=8)
    scale = np.abs(pos.vals) + 1e-6
    assert np.all(np.abs(got[m] - ref["G"].vals[m]) <= tol * scale[m])
    assert np.all(got[~m] == 0)
    np.testing.assert_allclose(st.gc.cpu().numpy(), ref["gc"], rtol=0, atol=tol)
    np.testing.assert_allclose(st.gb.cpu().numpy(), ref["gb"], rtol=0, atol=tol)


def test_fused_arithmetic_is_bit_identical_on_binary_operands():
    """All three products of the step multiply the weights by 0/1 samples, so every product is exact
    and the fused (FAST) arithmetic must give the same bits as the EXACT one and as the oracle."""
    import cuv_b200 as cb
    units, nd, nb = 2048, 128, 160
    offs = np.arange(-nd // 2, nd // 2, dtype=np.int32)
    W, V0, U_h, U_v = rbm_oracle.make_inputs(1005, units, units, offs, nb, w_std=0.05)
    exact = run_gpu_step(cb, W, V0, U_h, U_v, mode=cb.MODE_EXACT)
    fast = run_gpu_step(cb, W, V0, U_h, U_v, mode=cb.MODE_FAST)
    for name in ("H0p", "H0", "V1p", "V1", "H1p"):
        assert_bits_equal(cb.to_host(getattr(fast, name)), cb.to_host(getattr(exact, name)), name)
    assert_bits_equal(fast.G.vec.cpu().numpy(), exact.G.vec.cpu().numpy(), "G")
    # and the raw products equal the oracle's bit for bit in FAST mode
    Wd = cb.dev_dia_matrix_f(W.h, W.w, W.offsets, W.stride, W.rf).set_vec(W.vals)
    X = cb.colmajor_empty(units, nb)
    cb.prod(X, Wd, cb.to_device(V0), "n", "n", 1.0, 0.0, cb.MODE_FAST)
    want = np.zeros((units, nb), dtype=np.float32, order="F")
    ho.prod(want, W, V0, "n", nthreads=8)
    assert_bits_equal(cb.to_host(X), want, "prod 'n' FAST vs oracle on 0/1 input")
    cb.prod(X, Wd, exact.H0, "t", "n", 1.0, 0.0, cb.MODE_FAST)
    ho.prod(want, W, cb.to_host(exact.H0), "t", nthreads=8)
    assert_bits_equal(cb.to_host(X), want, "prod 't' FAST vs oracle on 0/1 input")


def test_sharded_partials_sum_to_full_batch():
    """Two column shards computed with the global batch in the factors add up to the unsharded step
    (what the all-reduce does across ranks), here on one GPU."""
    import cuv_b200 as cb
    from cuv_b200 import rbm
    units, nd, B = 1024, 64, 128
    offs = np.arange(-nd // 2, nd // 2, dtype=np.int32)
    W, V0, U_h, U_v = rbm_oracle.make_inputs(1004, units, units, offs, B, w_std=0.05)
    full = run_gpu_step(cb, W, V0, U_h, U_v)
    parts = []
    for r in range(2):
        c0, c1 = rbm.shard_columns(B, 2, r)
        sl = lambda a: np.asfortranarray(a[:, c0:c1])
        parts.append(run_gpu_step(cb, W, sl(V0), sl(U_h), sl(U_v), batch_global=B))
    G = parts[0].G.vec + parts[1].G.vec
    bias = parts[0].bias_grad + parts[1].bias_grad
    np.testing.assert_allclose(G.cpu().numpy(), full.G.vec.cpu().numpy(), rtol=0, atol=2e-6)
    np.testing.assert_allclose(bias.cpu().numpy(), full.bias_grad.cpu().numpy(), rtol=0, atol=2e-6)
    assert_bits_equal(cb.to_host(parts[1].H0p), np.asfortranarray(cb.to_host(full.H0p)[:, 64:]))


def test_host_fed_pipeline_matches_direct_step():
    """HostFedRBM (pinned host inputs, overlapped copies, gradients read back) gives the bits of the
    direct device-resident step, for consecutive steps on different inputs."""
    import torch
    import cuv_b200 as cb
    from cuv_b200 import rbm
    units, nd, nb = 1024, 64, 96
    offs = np.arange(-nd // 2, nd // 2, dtype=np.int32)
    sets = [rbm_oracle.make_inputs(2000 + i, units, units, offs, nb, w_std=0.05) for i in range(3)]
    W = sets[0][0]
    Wd = cb.dev_dia_matrix_f(W.h, W.w, W.offsets, W.stride, W.rf).set_vec(W.vals)
    direct = rbm.SparseRBMStep(Wd, nb)
    want = []
    for _, V0, U_h, U_v in sets:
        direct.step(cb.to_device(V0), cb.to_device(U_h), cb.to_device(U_v))
        want.append((direct.G.vec.cpu().numpy().copy(), direct.bias_grad.cpu().numpy().copy()))
    st = rbm.SparseRBMStep(Wd, nb)
    fed = rbm.HostFedRBM(st)
    pin = lambda a: torch.from_numpy(np.ascontiguousarray(a.T)).pin_memory()
    hosts = [tuple(pin(a) for a in s[1:]) for s in sets]
    outs = [(torch.empty(st.G.vec.numel()).pin_memory(), torch.empty(st.bias_grad.numel()).pin_memory()) for _ in sets]
    fed.submit(*hosts[0])
    for i in range(3):
        if i + 1 < 3:
            fed.submit(*hosts[i + 1])
        fed.run(*outs[i])
    fed.wait()
    torch.cuda.synchronize()
    for i in range(3):
        assert_bits_equal(outs[i][0].numpy(), want[i][0], "G of step %d" % i)
        assert_bits_equal(outs[i][1].numpy(), want[i][1], "bias gradients of step %d" % i)


@pytest.mark.parametrize("units,nd,nb", [(1024, 64, 96), (1000, 37, 50), (1001, 37, 50)])
def test_combined_entry_point_gives_the_bits_of_the_separate_calls(units, nd, nb):
    """The combined entry point (product + bias/logistic/compare) == prod followed by the element-wise
    call, bit for bit, on shapes that reach the banded and the windowed kernels."""
    import cuv_b200 as cb
    offs = np.arange(-(nd // 2), nd - nd // 2, dtype=np.int32)
    W, V0, U_h, U_v = rbm_oracle.make_inputs(3000 + nd, units, units, offs, nb, w_std=0.05)
    a = run_gpu_step(cb, W, V0, U_h, U_v, fused=True)
    b = run_gpu_step(cb, W, V0, U_h, U_v, fused=False)
    for name in ("H0p", "H0", "V1p", "V1", "H1p"):
        assert_bits_equal(cb.to_host(getattr(a, name)), cb.to_host(getattr(b, name)), name)
    assert_bits_equal(a.G.vec.cpu().numpy(), b.G.vec.cpu().numpy(), "G")
    assert_bits_equal(a.bias_grad.cpu().numpy(), b.bias_grad.cpu().numpy(), "bias gradients")


def test_update_step_applies_the_gradients():
    """updateStep of the trainer (examples/rbm/base.py:72-75): after a step, learn_step_weight_decay on the weight
    diagonals and both biases equals the host loop applied to the GPU's own gradients, bit for bit, and the next
    step runs on the updated weights."""
    import cuv_b200 as cb
    units, nd, nb = 1024, 32, 96
    offs = np.arange(-nd // 2, nd // 2, dtype=np.int32)
    W, V0, U_h, U_v = rbm_oracle.make_inputs(1006, units, units, offs, nb, w_std=0.05)
    st = run_gpu_step(cb, W, V0, U_h, U_v)
    w0, g = st.W.vec.cpu().numpy().copy(), st.G.vec.cpu().numpy().copy()
    c0, b0 = st.c_hid.cpu().numpy().copy(), st.b_vis.cpu().numpy().copy()
    gc, gb = st.gc.cpu().numpy().copy(), st.gb.cpu().numpy().copy()
    st.update(0.1, 0.002)
    assert_bits_equal(st.W.vec.cpu().numpy(), ho.learn_step_weight_decay(w0, g, 0.1, 0.002), "W")
    assert_bits_equal(st.c_hid.cpu().numpy(), ho.learn_step_weight_decay(c0, gc, 0.1, 0.002), "bias_hi")
    assert_bits_equal(st.b_vis.cpu().numpy(), ho.learn_step_weight_decay(b0, gb, 0.1, 0.002), "bias_lo")
    # second step on the updated model against the oracle's step on the same updated model (the hidden
    # probabilities do not depend on samples, so no tie between a probability and a uniform can matter)
    W2 = ho.DiaHost(W.h, W.w, W.offsets, W.stride, 1, st.W.vec.cpu().numpy())
    ref = rbm_oracle.cd1_step(W2, V0, U_h, U_v, b=st.b_vis.cpu().numpy(), c=st.c_hid.cpu().numpy(), nthreads=8)
    st.step(cb.to_device(V0), cb.to_device(U_h), cb.to_device(U_v))
    np.testing.assert_allclose(cb.to_host(st.H0p), ref["H0p"], rtol=1e-5)


def test_step_replayed_from_a_cuda_graph():
    """A step recorded into a CUDA graph (after one ordinary step has made the library allocate its scratch) replays
    with the same bits, also on new contents of the same input tensors."""
    import torch
    import cuv_b200 as cb
    from cuv_b200 import rbm
    units, nd, nb = 1024, 64, 128
    offs = np.arange(-nd // 2, nd // 2, dtype=np.int32)
    W, V0, U_h, U_v = rbm_oracle.make_inputs(1007, units, units, offs, nb, w_std=0.05)
    Wd = cb.dev_dia_matrix_f(W.h, W.w, W.offsets, W.stride, W.rf).set_vec(W.vals)
    st = rbm.SparseRBMStep(Wd, nb)
    dV0, dUh, dUv = cb.to_device(V0), cb.to_device(U_h), cb.to_device(U_v)
    graph = st.capture(dV0, dUh, dUv)
    eager = {k: getattr(st, k).clone() for k in ("H0p", "H0", "V1p", "V1", "H1p")}
    g_eager, b_eager = st.G.vec.clone(), st.bias_grad.clone()
    st.G.vec.zero_(); st.bias_grad.zero_(); st.H1p.zero_()
    graph.replay()
    torch.cuda.synchronize()
    for k, v in eager.items():
        assert torch.equal(getattr(st, k), v), k
    assert torch.equal(st.G.vec, g_eager) and torch.equal(st.bias_grad, b_eager)
    # new data in the same tensors: the replay follows it
    _, V0b, U_hb, U_vb = rbm_oracle.make_inputs(1008, units, units, offs, nb, w_std=0.05)
    dV0.copy_(cb.to_device(V0b)); dUh.copy_(cb.to_device(U_hb)); dUv.copy_(cb.to_device(U_vb))
    graph.replay()
    torch.cuda.synchronize()
    replayed = st.G.vec.clone()
    st.step(dV0, dUh, dUv)
    torch.cuda.synchronize()
    assert torch.equal(st.G.vec, replayed)
