"""The sharded CD-1 step on two GPUs: the CUDA kernels on each rank's batch columns plus the NCCL sum of the partial
gradients (through the C ABI: cuvdia_rbm_cd1_step_f32, cuvdia_nccl_comm_create, cuvdia_allreduce_grad) against the
unsharded step on one GPU and against the CPU oracle, all from ONE seeded input set sliced by shard_columns.
Skipped when fewer than two GPUs are visible."""
import os
import socket

import numpy as np
import pytest

from oracle import host_oracle as ho
from oracle import rbm_oracle

pytestmark = pytest.mark.gpu

UNITS, ND, B, SEED = 2048, 128, 256, 1021


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _inputs():
    offs = np.arange(-ND // 2, ND // 2, dtype=np.int32)
    return rbm_oracle.make_inputs(SEED, UNITS, UNITS, offs, B, w_std=0.05, nthreads=4)


def _rank_main(rank, world, port, out_dir):
    import torch
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    import cuv_b200 as cb
    from cuv_b200 import rbm
    W, V0, U_h, U_v = _inputs()
    c0, c1 = rbm.shard_columns(B, world, rank)
    sl = lambda a: cb.to_device(np.asfortranarray(a[:, c0:c1]), dev)
    Wd = cb.dev_dia_matrix_f(W.h, W.w, W.offsets, W.stride, W.rf, device=dev).set_vec(W.vals)
    st = rbm.SparseRBMStep(Wd, c1 - c0, B, cb.MODE_EXACT, dev)
    for _ in range(2):                       # twice: the collective leaves the same sum again on fresh partials
        st.step(sl(V0), sl(U_h), sl(U_v))
        st.allreduce()
    torch.cuda.synchronize()
    np.save(os.path.join(out_dir, "g%d.npy" % rank), st.G.vec.cpu().numpy())
    np.save(os.path.join(out_dir, "b%d.npy" % rank), st.bias_grad.cpu().numpy())
    np.save(os.path.join(out_dir, "h%d.npy" % rank), cb.to_host(st.H1p))
    assert cb.plan_status(Wd) == 0
    # the same sum over torch.distributed's own communicator: the two routes must agree bit for bit
    st.step(sl(V0), sl(U_h), sl(U_v))
    rbm.allreduce_gradients(st.G.vec, st.bias_grad)
    torch.cuda.synchronize()
    np.save(os.path.join(out_dir, "t%d.npy" % rank), st.G.vec.cpu().numpy())
    # and the one-call form that hides part of the collective under the step's last kernel
    st.grad_buf.zero_()
    st.step_allreduce(sl(V0), sl(U_h), sl(U_v))
    torch.cuda.synchronize()
    np.save(os.path.join(out_dir, "o%d.npy" % rank), st.grad_buf.cpu().numpy())
    assert cb.plan_status(Wd) == 0
    # the cut itself (forced: at this size it would cost a wave of blocks) on a band of five column tiles
    offs5 = np.arange(-256, 256, dtype=np.int32)
    W5, V5, Uh5, Uv5 = rbm_oracle.make_inputs(SEED + 1, UNITS, UNITS, offs5, B, w_std=0.02, nthreads=4)
    W5d = cb.dev_dia_matrix_f(W5.h, W5.w, W5.offsets, W5.stride, W5.rf, device=dev).set_vec(W5.vals)
    s5 = rbm.SparseRBMStep(W5d, c1 - c0, B, cb.MODE_EXACT, dev)
    s5._reducer = st._reducer
    s5.grad_buf.fill_(float("nan"))          # cells outside the diagonals' ranges are never written: they stay NaN
    s5.step(sl(V5), sl(Uh5), sl(Uv5))
    s5.allreduce()
    torch.cuda.synchronize()
    plain = s5.grad_buf.cpu().numpy().copy()
    for _ in range(2):
        s5.grad_buf.fill_(float("nan"))
        s5.step_allreduce(sl(V5), sl(Uh5), sl(Uv5), overlap=2)
        torch.cuda.synchronize()
        np.save(os.path.join(out_dir, "c%d.npy" % rank), np.stack([plain, s5.grad_buf.cpu().numpy()]))
    assert cb.plan_status(W5d) == 0
    # the step that draws its uniform numbers on the device: every rank passes the global index of its first column
    st.grad_buf.zero_()
    st.step_drawn_allreduce(sl(V0), 77, 5, c0)
    torch.cuda.synchronize()
    np.save(os.path.join(out_dir, "d%d.npy" % rank), st.grad_buf.cpu().numpy())
    np.save(os.path.join(out_dir, "s%d.npy" % rank), cb.to_host(st.V1))
    st._reducer.close()
    dist.destroy_process_group()


def test_two_gpu_step_and_nccl_sum_equal_the_unsharded_step(tmp_path):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    import cuv_b200 as cb
    from cuv_b200 import rbm
    world = 2
    mp.spawn(_rank_main, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    W, V0, U_h, U_v = _inputs()
    g = [np.load(tmp_path / ("g%d.npy" % r)) for r in range(world)]
    b = [np.load(tmp_path / ("b%d.npy" % r)) for r in range(world)]
    assert np.array_equal(g[0], g[1]) and np.array_equal(b[0], b[1])         # every rank holds the same sum
    assert np.array_equal(np.load(tmp_path / "t0.npy"), g[0])
    for r in range(world):                                                    # the overlapped form: the same bits
        assert np.array_equal(np.load(tmp_path / ("o%d.npy" % r)), np.concatenate([g[r], b[r]]))
    for r in range(world):                                                    # ... also when the last kernel is cut in two
        plain, cut = np.load(tmp_path / ("c%d.npy" % r))
        m5 = np.isfinite(plain)
        assert np.array_equal(np.isfinite(cut), m5) and np.array_equal(cut[m5], plain[m5])
    # against the unsharded step on one GPU
    Wd = cb.dev_dia_matrix_f(W.h, W.w, W.offsets, W.stride, W.rf).set_vec(W.vals)
    full = rbm.SparseRBMStep(Wd, B, B, cb.MODE_EXACT)
    full.step(cb.to_device(V0), cb.to_device(U_h), cb.to_device(U_v))
    np.testing.assert_allclose(g[0], full.G.vec.cpu().numpy(), rtol=0, atol=2e-6)
    np.testing.assert_allclose(b[0], full.bias_grad.cpu().numpy(), rtol=0, atol=2e-6)
    H1p = np.concatenate([np.load(tmp_path / ("h%d.npy" % r)) for r in range(world)], axis=1)
    assert np.array_equal(H1p, cb.to_host(full.H1p))                          # the shards are the full batch's columns
    # the drawn-sample step: the shards draw what the unsharded run draws, and the oracle restates those numbers
    full.step_drawn(cb.to_device(V0), 77, 5, 0)
    d = [np.load(tmp_path / ("d%d.npy" % r)) for r in range(world)]
    assert np.array_equal(d[0], d[1])
    np.testing.assert_allclose(d[0], full.grad_buf.cpu().numpy(), rtol=0, atol=2e-6)
    V1 = np.concatenate([np.load(tmp_path / ("s%d.npy" % r)) for r in range(world)], axis=1)
    assert np.array_equal(V1, cb.to_host(full.V1))
    assert np.array_equal(V1, (cb.to_host(full.V1p) > ho.uniform(UNITS, B, 77, 5, 0, which=1)).astype(np.float32))
    # against the CPU oracle's unsharded step
    ref = rbm_oracle.cd1_step(W, V0, U_h, U_v, nthreads=8)
    tol = 1e-4 * np.sqrt(B / 128.0)
    m = ref["G"].valid_mask().reshape(-1)
    pos = ho.DiaHost(W.h, W.w, W.offsets, W.stride, 1)
    ho.densedense_to_dia(pos, ref["H0p"], V0, 1.0 / B, 0.0, nthreads=8)
    assert np.all(np.abs(g[0][m] - ref["G"].vals[m]) <= tol * (np.abs(pos.vals[m]) + 1e-6))
    assert np.all(g[0][~m] == 0)
    np.testing.assert_allclose(b[0], np.concatenate([ref["gc"], ref["gb"]]), rtol=0, atol=tol)
