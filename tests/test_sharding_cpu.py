"""Multi-GPU sharding logic on CPU: plan, local tile sets, gloo all-gather (world_size 2), assembly.

The local GEMM of each rank is played by the CPU oracle here (test stand-in only); what is under test
is the host logic every rank runs and the collective that joins the slabs.
"""
import os

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import masked_gemm as og
from tilesparsity_b200 import sharding, synth
from tilesparsity_b200.tiles import tile_bounds_from_col_mask, tiles_from_lists


def _problem():
    g = synth.rng(17)
    K, N, M = 96, 1000, 48
    col = g.random(N) < 0.8
    nt = len(tile_bounds_from_col_mask(col, 128)) - 1
    counts = synth.beta_skewed_counts(K, nt, 0.3, 5)
    lists = [np.sort(g.permutation(K)[:c]).astype(np.int32) for c in counts]
    ts = tiles_from_lists(K, N, 128, lists, col)
    A = g.standard_normal((M, K)).astype(np.float32)
    W = g.standard_normal((K, N)).astype(np.float32)
    return ts, A, W


def test_plan_covers_every_tile_once_and_balances():
    ts, _, _ = _problem()
    for world in (1, 2, 3, 8):
        p = sharding.plan(ts, world)
        assert sorted(np.concatenate([p.tiles_of(r) for r in range(world)]).tolist()) == list(range(ts.n_tiles))
        assert p.n_pad % 8 == 0 and p.n_pad >= max(p.n_local)
        order = sharding.column_order(ts, p)
        assert sorted(order[order >= 0].tolist()) == sorted(ts.kept_n.tolist())
        if world <= ts.n_tiles:
            assert p.load().max() <= p.load().sum() / world + p.cost.max()      # LPT bound
    assert sharding.plan(ts, 1).balance() == 1.0


def _worker(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        ts, A, W = _problem()
        p = sharding.plan(ts, world)
        local, gcols = sharding.local_tiles(ts, p, rank)
        slab = np.zeros((p.n_pad, A.shape[0]), dtype=np.float32)
        slab[:len(gcols)] = og.masked_matmul_compacted(A.T.copy(), W[:, gcols], local)[:len(gcols)]
        out = torch.empty((world * p.n_pad, A.shape[0]), dtype=torch.float32)
        dist.all_gather_into_tensor(out, torch.from_numpy(slab))
        full = sharding.assemble(out, sharding.column_order(ts, p), ts.N).numpy()
        ref = og.masked_matmul_compacted(A.T.copy(), W, ts)
        q.put((rank, float(np.abs(full - ref).max()), p.load().tolist()))
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(120)
def test_two_ranks_gather_the_full_output_over_gloo():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + (os.getpid() % 2000)
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for pr in procs:
        pr.start()
    res = [q.get(timeout=100) for _ in procs]
    for pr in procs:
        pr.join(timeout=30)
        assert pr.exitcode == 0
    assert sorted(r[0] for r in res) == [0, 1]
    assert all(r[1] < 1e-4 for r in res)
    assert res[0][2] == res[1][2]                   # both ranks computed the same plan
