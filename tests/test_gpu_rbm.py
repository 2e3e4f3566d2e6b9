"""The sparse-RBM CD-1 step on the GPU against the CPU oracle's step (same seeded inputs)."""
import numpy as np
import pytest

from oracle import host_oracle as ho
from oracle import rbm_oracle
from tests.helpers import assert_bits_equal

pytestmark = pytest.mark.gpu


def run_gpu_step(cb, W, V0, U_h, U_v, batch_global=None, mode=None, fused=False, **kw):
    from cuv_b200 import rbm
    Wd = cb.dev_dia_matrix_f(W.h, W.w, W.offsets, W.stride, W.rf).set_vec(W.vals)
    st = rbm.SparseRBMStep(Wd, V0.shape[1], batch_global, cb.MODE_EXACT if mode is None else mode, fused=fused, **kw)
    st.step(cb.to_device(V0), cb.to_device(U_h), cb.to_device(U_v))
    return st


# the step as one C call with the bias sums taken in the element-wise passes (default), and the trainer's literal
# call sequence with four reductions, through the combined product + element-wise entry point
STEP_VARIANTS = [dict(), dict(fused=True)]


@pytest.mark.parametrize("variant", STEP_VARIANTS, ids=["c_step", "combined_calls"])
@pytest.mark.parametrize("units,nd,nb", [(1024, 32, 96), (2048, 128, 160), (1000, 37, 50), (1001, 37, 50), (404, 28, 4),
                                         (953, 197, 2), (2953, 95, 19)])
def test_cd1_step_matches_oracle(units, nd, nb, variant):
    import cuv_b200 as cb
    offs = np.arange(-(nd // 2), nd - nd // 2, dtype=np.int32)
    W, V0, U_h, U_v = rbm_oracle.make_inputs(1003, units, units, offs, nb, w_std=0.05)
    ref = rbm_oracle.cd1_step(W, V0, U_h, U_v, nthreads=8)
    st = run_gpu_step(cb, W, V0, U_h, U_v, **variant)
    np.testing.assert_allclose(cb.to_host(st.H0p), ref["H0p"], rtol=1e-5)           # activations: rel 1e-5
    assert np.array_equal(cb.to_host(st.H0), ref["H0"])                              # samples identical
    np.testing.assert_allclose(cb.to_host(st.V1p), ref["V1p"], rtol=1e-5)
    assert np.array_equal(cb.to_host(st.V1), ref["V1"])
    np.testing.assert_allclose(cb.to_host(st.H1p), ref["H1p"], rtol=1e-5)
    # gradients are differences of two batch sums: compare against the size of the two summands (with a batch of a
    # few columns the positive sum of a cell is often exactly zero - no column has that visible unit on - while the
    # negative one is not)
    tol = 1e-4 * np.sqrt(max(nb, 128) / 128.0)
    m = ref["G"].valid_mask().reshape(-1)
    got = st.G.vec.cpu().numpy()
    pos, neg = ho.DiaHost(W.h, W.w, W.offsets, W.stride, 1), ho.DiaHost(W.h, W.w, W.offsets, W.stride, 1)
    ho.densedense_to_dia(pos, ref["H0p"], V0, 1.0 / nb, 0.0, nthreads=8)
    ho.densedense_to_dia(neg, ref["H1p"], ref["V1"], 1.0 / nb, 0.0, nthreads=8)
    scale = np.abs(pos.vals) + np.abs(neg.vals) + 1e-6
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
    b = run_gpu_step(cb, W, V0, U_h, U_v, fused=False, bias_sums="reduce")
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


@pytest.mark.parametrize("units,nb", [(1024, 96), (1000, 50), (4096, 7), (1027, 33), (8192, 1024)])
def test_elementwise_pass_with_batch_sums(units, nb):
    """bias + logistic + compare with the per-unit batch sum taken in the same pass: activations and samples are the
    bits of the plain pass, the sums agree with a float64 sum (activations) or are exact (0/1 samples), accumulate
    with factOld, and are identical run to run."""
    import torch
    import cuv_b200 as cb
    g = torch.Generator(device="cuda"); g.manual_seed(units + nb)
    mk = lambda lo, hi: cb.colmajor_empty(units, nb).uniform_(lo, hi, generator=g)
    pre, U = mk(-3, 3), mk(0, 1)
    bias = torch.empty(units, device="cuda").uniform_(-1, 1, generator=g)
    act0, S0 = pre.clone(), cb.colmajor_empty(units, nb)
    cb.bias_sigmoid_sample(act0, bias, U, S0)
    tol = 1e-4 * np.sqrt(max(nb, 128) / 128.0)
    for of_sample in (False, True):
        act, S = pre.clone(), cb.colmajor_empty(units, nb)
        dst = torch.full((units,), float("nan"), device="cuda")          # factOld == 0: never read
        cb.bias_sigmoid_sample_sum(act, bias, U, S, dst, of_sample, 0.25, 0.0)
        assert torch.equal(act, act0) and torch.equal(S, S0)
        want = (S0 if of_sample else act0).double().sum(dim=1) * 0.25
        if of_sample:
            assert torch.equal(dst.double(), want)
        else:
            assert float(((dst.double() - want).abs() / want.abs().clamp_min(1e-6)).max()) <= tol
        again = dst.clone()
        cb.bias_sigmoid_sample_sum(pre.clone(), bias, U, S, again, of_sample, 0.25, 0.0)
        assert torch.equal(again, dst)
        acc = torch.ones(units, device="cuda")
        cb.bias_sigmoid_sample_sum(pre.clone(), bias, U, S, acc, of_sample, -0.25, 2.0)
        np.testing.assert_allclose(acc.cpu().numpy(), (2.0 - dst).cpu().numpy(), rtol=1e-6, atol=1e-6)
    # store_act=False: samples and their sum as before, the activations left as they were
    act, S = pre.clone(), cb.colmajor_empty(units, nb)
    dst = torch.empty(units, device="cuda")
    cb.bias_sigmoid_sample_sum(act, bias, U, S, dst, True, 1.0, 0.0, store_act=False)
    assert torch.equal(act, pre) and torch.equal(S, S0) and torch.equal(dst.double(), S0.double().sum(dim=1))
    # no sampling: activations only, no bias
    act, act1 = pre.clone(), pre.clone()
    cb.bias_sigmoid_sample(act1)
    cb.bias_sigmoid_sample_sum(act, None, None, None, dst, False, 1.0, 0.0)
    assert torch.equal(act, act1)
    assert float(((dst.double() - act1.double().sum(dim=1)).abs() / act1.double().sum(dim=1)).max()) <= tol


def test_c_step_equals_the_call_by_call_step():
    """cuvdia_rbm_cd1_step_f32 queues exactly the launches of forward() + gradients(): same bits everywhere; the
    bias sums taken in the element-wise passes agree with the four separate reductions within the batch-sum
    tolerance, and keep_v1p=False changes nothing but V1p."""
    import cuv_b200 as cb
    from cuv_b200 import rbm
    units, nd, nb = 2048, 96, 224
    offs = np.arange(-nd // 2, nd // 2, dtype=np.int32)
    W, V0, U_h, U_v = rbm_oracle.make_inputs(1011, units, units, offs, nb, w_std=0.05)
    b = (np.random.default_rng(3).standard_normal(units) * 0.1).astype(np.float32)
    c = (np.random.default_rng(4).standard_normal(units) * 0.1).astype(np.float32)
    dV0, dUh, dUv = cb.to_device(V0), cb.to_device(U_h), cb.to_device(U_v)

    def make(**kw):
        Wd = cb.dev_dia_matrix_f(W.h, W.w, W.offsets, W.stride, W.rf).set_vec(W.vals)
        st = rbm.SparseRBMStep(Wd, nb, 4 * nb, **kw)
        st.b_vis.copy_(cb.to_device(b)); st.c_hid.copy_(cb.to_device(c))
        return st
    one = make(); one.step(dV0, dUh, dUv)
    calls = make(); calls.forward(dV0, dUh, dUv); calls.gradients(dV0)
    for name in ("H0p", "H0", "V1p", "V1", "H1p"):
        assert_bits_equal(cb.to_host(getattr(one, name)), cb.to_host(getattr(calls, name)), name)
    assert_bits_equal(one.G.vec.cpu().numpy(), calls.G.vec.cpu().numpy(), "G")
    assert_bits_equal(one.bias_grad.cpu().numpy(), calls.bias_grad.cpu().numpy(), "bias gradients")
    sep = make(bias_sums="reduce"); sep.step(dV0, dUh, dUv)
    assert_bits_equal(one.G.vec.cpu().numpy(), sep.G.vec.cpu().numpy(), "G vs separate reductions")
    tol = 1e-4 * np.sqrt(max(nb, 128) / 128.0)
    np.testing.assert_allclose(one.bias_grad.cpu().numpy(), sep.bias_grad.cpu().numpy(), rtol=0, atol=tol)
    lean = make(keep_v1p=False); lean.step(dV0, dUh, dUv)
    for name in ("H0p", "H0", "V1", "H1p"):
        assert_bits_equal(cb.to_host(getattr(lean, name)), cb.to_host(getattr(one, name)), name)
    assert_bits_equal(lean.grad_buf.cpu().numpy(), one.grad_buf.cpu().numpy(), "gradients without V1p written")
    ref = rbm_oracle.cd1_step(W, V0, U_h, U_v, batch_global=4 * nb, b=b, c=c, nthreads=8)
    np.testing.assert_allclose(one.gc.cpu().numpy(), ref["gc"], rtol=0, atol=tol)
    np.testing.assert_allclose(one.gb.cpu().numpy(), ref["gb"], rtol=0, atol=tol)


def test_cd1_step_at_config3_size():
    """BASELINE config 3 (16384 units, 512 diagonals, batch 1024) through the one-call step: the activations of a
    16-column slice against the oracle (the oracle's step on those columns; samples identical because uniforms
    that tie with a probability are moved away first), the bias gradients against float64 sums, and the weight
    gradient through three diagonals computed by the oracle on all columns and the trace identity
    sum(G * W) == (<H0p, W V0> - <H1p, W V1>) / B."""
    import torch
    import cuv_b200 as cb
    from cuv_b200 import rbm
    units, nd, nb = 16384, 512, 1024
    offs = np.arange(-nd // 2, nd // 2, dtype=np.int32)
    g = torch.Generator(device="cuda"); g.manual_seed(1003)
    Wd = cb.dev_dia_matrix_f(units, units, offs, units, 1)
    Wd.vec.normal_(0.0, 0.01, generator=g)
    mask = torch.from_numpy(ho.DiaHost(units, units, offs, units, 1).valid_mask().reshape(-1)).cuda()
    Wd.vec[~mask] = 0.0
    V0 = cb.colmajor_empty(units, nb); V0.t().copy_((torch.rand((nb, units), device="cuda", generator=g) < 0.3).float())
    U_h, U_v = cb.colmajor_empty(units, nb), cb.colmajor_empty(units, nb)
    U_h.t().copy_(torch.rand((nb, units), device="cuda", generator=g))
    U_v.t().copy_(torch.rand((nb, units), device="cuda", generator=g))
    st = rbm.SparseRBMStep(Wd, nb, mode=cb.MODE_FAST)

    def away(p, u):          # uniforms within 1e-4 of their probability move 1e-3 away (rbm_oracle.make_inputs does the same)
        near = (p - u).abs() < 1e-4
        u[near] = torch.where(p[near] >= 0.5, p[near] - 1e-3, p[near] + 1e-3)
    st.step(V0, U_h, U_v); away(st.H0p, U_h)
    st.step(V0, U_h, U_v); away(st.V1p, U_v)
    st.step(V0, U_h, U_v)
    cols = list(range(0, nb, nb // 16))
    Wh = ho.DiaHost(units, units, offs, units, 1, Wd.vec.cpu().numpy())
    sl = lambda t: np.asfortranarray(t[:, cols].cpu().numpy())
    ref = rbm_oracle.cd1_step(Wh, sl(V0), sl(U_h), sl(U_v), batch_global=nb, nthreads=8)
    np.testing.assert_allclose(sl(st.H0p), ref["H0p"], rtol=1e-5)
    assert np.array_equal(sl(st.H0), ref["H0"])
    np.testing.assert_allclose(sl(st.V1p), ref["V1p"], rtol=1e-5)
    assert np.array_equal(sl(st.V1), ref["V1"])
    np.testing.assert_allclose(sl(st.H1p), ref["H1p"], rtol=1e-5)
    tol = 1e-4 * np.sqrt(nb / 128.0)
    want_gc = (st.H0p.double().sum(dim=1) - st.H1p.double().sum(dim=1)) / nb
    want_gb = (V0.double().sum(dim=1) - st.V1.double().sum(dim=1)) / nb
    assert float((st.gc.double() - want_gc).abs().max()) <= tol
    assert float((st.gb.double() - want_gb).abs().max()) <= tol
    some = [0, nd // 2, nd - 1]
    pos, neg = ho.DiaHost(units, units, offs[some], units, 1), ho.DiaHost(units, units, offs[some], units, 1)
    full = lambda t: np.asfortranarray(t.cpu().numpy())
    ho.densedense_to_dia(pos, full(st.H0p), full(V0), 1.0 / nb, 0.0, nthreads=8)
    ho.densedense_to_dia(neg, full(st.H1p), full(st.V1), 1.0 / nb, 0.0, nthreads=8)
    got = st.G.vec.cpu().numpy().reshape(nd, units)[some]
    m = pos.valid_mask()
    p_, n_ = pos.vals.reshape(len(some), units), neg.vals.reshape(len(some), units)
    assert np.all(np.abs(got[m] - (p_[m] - n_[m])) <= tol * (np.abs(p_[m]) + 1e-6))
    WV0, WV1 = cb.colmajor_empty(units, nb), cb.colmajor_empty(units, nb)
    cb.prod(WV0, Wd, V0, "n"); cb.prod(WV1, Wd, st.V1, "n")
    dot = lambda a, b_: float((a.double() * b_.double()).sum().item())
    lhs = float((st.G.vec.double() * Wd.vec.double()).sum().item())
    rhs = (dot(st.H0p, WV0) - dot(st.H1p, WV1)) / nb
    scale = (dot(st.H0p, WV0.abs()) + dot(st.H1p, WV1.abs())) / nb
    assert abs(lhs - rhs) <= 1e-5 * scale


@pytest.mark.parametrize("rows,ncols,ld_pad", [(1024, 33, 0), (1001, 7, 3), (6, 5, 0)])
def test_device_drawn_uniforms_equal_the_oracle(rows, ncols, ld_pad):
    """cuvdia_uniform_f32 against the CPU restatement of the generator, bit for bit, with a column offset (what a
    rank that holds a shard of the batch passes) and a padded leading dimension."""
    import cuv_b200 as cb
    buf = cb.colmajor_empty(rows + ld_pad, ncols)
    buf.fill_(-1.0)
    cb.fill_rnd_uniform(buf[:rows], seed=0x1234567890abcdef, step=3, col0=2 ** 33 + 5, which=1)
    want = ho.uniform(rows, ncols, seed=0x1234567890abcdef, step=3, col0=2 ** 33 + 5, which=1)
    assert_bits_equal(cb.to_host(buf[:rows]), want, "uniform numbers")
    if ld_pad:
        assert (buf[rows:] == -1.0).all()


@pytest.mark.parametrize("rows,ncols,ld_pad", [(1024, 33, 0), (1001, 7, 3), (6, 5, 0)])
def test_rnd_binarize_equals_the_compare_with_the_oracles_numbers(rows, ncols, ld_pad):
    """cuvdia_rnd_binarize_f32 (CUV's rnd_binarize): in place, 1 where the activation exceeds the generator's number
    of that element and 0 elsewhere, rows beyond the matrix in a padded leading dimension untouched."""
    import cuv_b200 as cb
    rng = np.random.default_rng(rows * 31 + ncols)
    act = np.asfortranarray(rng.random((rows, ncols), dtype=np.float32))
    act[rng.random((rows, ncols)) < 0.05] = 0.0                       # 0 > u never holds, u = 0 included
    act[rng.random((rows, ncols)) < 0.05] = 1.0                       # 1 > u always holds
    buf = cb.colmajor_empty(rows + ld_pad, ncols)
    buf.fill_(-7.0)
    buf[:rows].copy_(cb.to_device(act))
    cb.rnd_binarize(buf[:rows], seed=42, step=9, col0=12345, which=1)
    u = ho.uniform(rows, ncols, seed=42, step=9, col0=12345, which=1)
    assert_bits_equal(cb.to_host(buf[:rows]), (act > u).astype(np.float32), "binarised activation")
    if ld_pad:
        assert (buf[rows:] == -7.0).all()


@pytest.mark.parametrize("units,nd,nb", [(1024, 64, 96), (1001, 37, 50)])
def test_step_with_drawn_samples_equals_the_step_on_those_numbers(units, nd, nb):
    """The step that draws its uniform numbers inside the element-wise passes gives, bit for bit, the step that reads
    them from memory when those tensors hold the same numbers - which the oracle produces too - so every parity check
    of the precomputed-number step carries over; with a column shard (col0) as a rank of a sharded run passes it."""
    import cuv_b200 as cb
    from cuv_b200 import rbm
    offs = np.arange(-(nd // 2), nd - nd // 2, dtype=np.int32)
    W, V0, _, _ = rbm_oracle.make_inputs(1009, units, units, offs, nb, w_std=0.05)
    seed, step, col0 = 99, 4, 1000
    U_h = ho.uniform(units, nb, seed, step, col0, which=0)
    U_v = ho.uniform(units, nb, seed, step, col0, which=1)
    ref = run_gpu_step(cb, W, V0, U_h, U_v, mode=cb.MODE_FAST)
    Wd = cb.dev_dia_matrix_f(W.h, W.w, W.offsets, W.stride, W.rf).set_vec(W.vals)
    st = rbm.SparseRBMStep(Wd, nb, None, cb.MODE_FAST)
    st.step_drawn(cb.to_device(V0), seed, step, col0)
    for name in ("H0p", "H0", "V1p", "V1", "H1p"):
        assert_bits_equal(cb.to_host(getattr(st, name)), cb.to_host(getattr(ref, name)), name)
    assert_bits_equal(st.G.vec.cpu().numpy(), ref.G.vec.cpu().numpy(), "G")
    assert_bits_equal(st.bias_grad.cpu().numpy(), ref.bias_grad.cpu().numpy(), "bias gradients")
    # and the samples are the oracle's comparison of the GPU's probabilities with the oracle's numbers
    assert np.array_equal(cb.to_host(st.H0), (cb.to_host(st.H0p) > U_h).astype(np.float32))
    assert np.array_equal(cb.to_host(st.V1), (cb.to_host(st.V1p) > U_v).astype(np.float32))
