"""The multi-rank path on CPU ranks (gloo, world size 2): batch-column sharding plus the gradient
all-reduce of cuv_b200.rbm, with the per-rank partial gradients produced by the CPU oracle."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import host_oracle as ho
from oracle import rbm_oracle

UNITS, ND, B = 256, 16, 32


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _rank_main(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from cuv_b200 import rbm
    offs = np.arange(-ND // 2, ND // 2, dtype=np.int32)
    W, V0, U_h, U_v = rbm_oracle.make_inputs(77, UNITS, UNITS, offs, B, w_std=0.05, nthreads=1)
    c0, c1 = rbm.shard_columns(B, world, rank)
    sl = lambda a: np.asfortranarray(a[:, c0:c1])
    part = rbm_oracle.cd1_step(W, sl(V0), sl(U_h), sl(U_v), batch_global=B)
    g = torch.from_numpy(part["G"].vals.copy())
    bias = torch.from_numpy(np.concatenate([part["gc"], part["gb"]]))
    rbm.allreduce_gradients(g, bias)
    np.save(os.path.join(out_dir, "g%d.npy" % rank), g.numpy())
    np.save(os.path.join(out_dir, "b%d.npy" % rank), bias.numpy())
    # the same with the samples' uniform numbers drawn from the generator: a rank passes the global index of its first
    # column and so draws the numbers the unsharded run draws for those columns
    Uh = ho.uniform(UNITS, c1 - c0, seed=5, step=2, col0=c0, which=0)
    Uv = ho.uniform(UNITS, c1 - c0, seed=5, step=2, col0=c0, which=1)
    part = rbm_oracle.cd1_step(W, sl(V0), Uh, Uv, batch_global=B)
    g = torch.from_numpy(part["G"].vals.copy())
    bias = torch.from_numpy(np.concatenate([part["gc"], part["gb"]]))
    rbm.allreduce_gradients(g, bias)
    np.save(os.path.join(out_dir, "dg%d.npy" % rank), g.numpy())
    np.save(os.path.join(out_dir, "ds%d.npy" % rank), part["V1"])
    dist.destroy_process_group()


def test_two_rank_allreduce_equals_unsharded_step(tmp_path):
    world = 2
    mp.spawn(_rank_main, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    offs = np.arange(-ND // 2, ND // 2, dtype=np.int32)
    W, V0, U_h, U_v = rbm_oracle.make_inputs(77, UNITS, UNITS, offs, B, w_std=0.05, nthreads=1)
    full = rbm_oracle.cd1_step(W, V0, U_h, U_v)
    g0, g1 = np.load(tmp_path / "g0.npy"), np.load(tmp_path / "g1.npy")
    assert np.array_equal(g0, g1)                                  # every rank ends with the same sum
    np.testing.assert_allclose(g0, full["G"].vals, rtol=0, atol=2e-6)
    b0 = np.load(tmp_path / "b0.npy")
    np.testing.assert_allclose(b0, np.concatenate([full["gc"], full["gb"]]), rtol=0, atol=2e-6)
    # drawn samples: the shards' numbers are the unsharded run's, so the samples are its columns and the sums agree
    Uh, Uv = ho.uniform(UNITS, B, seed=5, step=2, col0=0, which=0), ho.uniform(UNITS, B, seed=5, step=2, col0=0, which=1)
    full = rbm_oracle.cd1_step(W, V0, Uh, Uv)
    V1 = np.concatenate([np.load(tmp_path / ("ds%d.npy" % r)) for r in range(world)], axis=1)
    assert np.array_equal(V1, full["V1"])
    np.testing.assert_allclose(np.load(tmp_path / "dg0.npy"), full["G"].vals, rtol=0, atol=2e-6)


def test_shard_columns():
    from cuv_b200 import rbm
    assert [rbm.shard_columns(8192, 8, r) for r in (0, 7)] == [(0, 1024), (7168, 8192)]
    with pytest.raises(ValueError):
        rbm.shard_columns(10, 4, 0)
