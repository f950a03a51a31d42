"""Tile-sharded layer on real GPUs (needs at least two): NCCL all-gather and the fused
GEMM + all-gather (epilogue stores into peer-mapped buffers) against the unsharded layer."""
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, q):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from tilesparsity_b200 import TWLayer, sharding, synth
        from tilesparsity_b200.tiles import tiles_from_lists
        g = synth.rng(33)
        K, N, M = 512, 1536, 776
        counts = synth.beta_skewed_counts(K, N // 128, 0.3, 9)
        lists = [np.sort(g.permutation(K)[:c]).astype(np.int32) for c in counts]
        ts = tiles_from_lists(K, N, 128, lists)
        W = torch.from_numpy((g.standard_normal((K, N), dtype=np.float32) * 0.05)).to(dev)
        At = torch.from_numpy(g.standard_normal((K, M), dtype=np.float32)).to(dev, torch.float16)
        full = TWLayer(ts, torch.float16, dev)
        full.pack(W)
        ref = full.masked_gemm(At)
        shard = sharding.ShardedTWLayer(W, ts, rank, world, torch.float16)
        # NCCL path
        gathered = shard.all_gather(shard.masked_gemm(At))
        ok_nccl = torch.equal(shard.assemble(gathered), ref)
        # fused path, twice in a row on the same buffer
        buf, handle = shard.make_gather_buffer(M)
        ok_fused = True
        for scale in (1.0, 2.0):
            out = shard.masked_gemm_allgather(At * scale, buf, handle)
            want = full.masked_gemm(At * scale)
            ok_fused = ok_fused and torch.equal(shard.assemble(out), want)
        # the same through the NVSwitch multicast mapping of the buffer, where the box has one
        ok_mc = True
        if shard.has_multicast(handle):
            for scale in (3.0, 1.0):
                out = shard.masked_gemm_allgather(At * scale, buf, handle, multicast=True)
                ok_mc = ok_mc and torch.equal(shard.assemble(out), full.masked_gemm(At * scale))
        torch.cuda.synchronize()
        q.put((rank, bool(ok_nccl), bool(ok_fused), bool(ok_mc)))
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(300)
def test_sharded_layer_nccl_and_fused_allgather():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29700 + (os.getpid() % 1000)
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=240) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert all(r[1] for r in res), "NCCL all-gather path differs from the unsharded layer"
    assert all(r[2] for r in res), "fused GEMM + all-gather differs from the unsharded layer"
    assert all(r[3] for r in res), "fused GEMM + multicast all-gather differs from the unsharded layer"
