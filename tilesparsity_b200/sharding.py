"""Multi-GPU path: column tiles sharded across the GPUs of one box, balanced by kept FLOPs.

The reference has no multi-device code; its unit of distribution is the column tile, one per CUDA
stream (StreamMaskedGEMM/perf/basic_nn.cu:396-427).  Tiles are independent (tile t reads the kept
rows of At and its own packed weights and writes its own columns of C; nothing is reduced across
tiles), so the same unit shards across GPUs with no data-path collective:

* `plan` assigns tiles to ranks by greedy longest-processing-time on K_t * N_t (`ts_shard_plan`);
* every rank packs only its own tiles (weights stay resident per GPU), keeps a replica of the
  activations At, and writes a compact slab Ct_local[n_local, M] holding its kept columns in tile order;
* `all_gather` (NCCL over NVLink, or gloo on CPU in the tests) assembles the slabs only when the
  consumer needs the whole output; `column_order` tells which global column each gathered row is, so
  a following masked layer can absorb the permutation into its kept-row lists instead of moving data.

One process per GPU (`torch.distributed`); the plan is a pure host function, so every rank computes
the same plan without communicating.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import numpy as np

from ._lib import check, lib
from .tiles import TileSet


@dataclass
class ShardPlan:
    world: int
    owner: np.ndarray          # [n_tiles] rank that owns each tile
    cost: np.ndarray           # [n_tiles] K_t * N_t
    n_local: list              # kept columns per rank
    n_pad: int                 # slab rows every rank allocates (max over ranks, rounded up to 8)

    def tiles_of(self, rank: int) -> np.ndarray:
        return np.flatnonzero(self.owner == rank)

    def load(self) -> np.ndarray:
        return np.asarray([int(self.cost[self.owner == r].sum()) for r in range(self.world)], dtype=np.int64)

    def balance(self) -> float:
        ld = self.load()
        return float(ld.mean() / ld.max()) if ld.max() > 0 else 1.0


def plan(tiles: TileSet, world: int) -> ShardPlan:
    """Tile -> rank assignment, identical on every rank."""
    cost = (tiles.k_counts().astype(np.int64) * tiles.n_counts().astype(np.int64))
    owner = np.zeros(max(tiles.n_tiles, 1), dtype=np.int32)
    if tiles.n_tiles:
        check(lib.ts_shard_plan(tiles.n_tiles, cost.ctypes.data_as(C.POINTER(C.c_int64)), world,
                                owner.ctypes.data_as(C.POINTER(C.c_int32))))
    owner = owner[:tiles.n_tiles]
    n_local = [int(tiles.n_counts()[owner == r].sum()) for r in range(world)]
    n_pad = (max(n_local + [1]) + 7) // 8 * 8
    return ShardPlan(world, owner, cost, n_local, n_pad)


def local_tiles(tiles: TileSet, p: ShardPlan, rank: int):
    """The rank's share as a TileSet over its own compact column space, plus the global column of
    every local column (tile order, ascending inside a tile)."""
    mine = p.tiles_of(rank)
    cols = [tiles.tile_cols(t) for t in mine]
    rows = [tiles.tile_rows(t) for t in mine]
    n_local = int(sum(len(c) for c in cols))
    kp = np.concatenate([[0], np.cumsum([len(r) for r in rows])]).astype(np.int32)
    npz = np.concatenate([[0], np.cumsum([len(c) for c in cols])]).astype(np.int32)
    global_cols = np.concatenate(cols).astype(np.int32) if cols else np.zeros(0, np.int32)
    kept_k = np.concatenate(rows).astype(np.int32) if rows else np.zeros(0, np.int32)
    local = TileSet(tiles.K, max(n_local, 1), tiles.G, npz.copy(), kp, kept_k, npz,
                    np.arange(n_local, dtype=np.int32))
    return local, global_cols


def column_order(tiles: TileSet, p: ShardPlan) -> np.ndarray:
    """Global column held by each row of the gathered [world * n_pad, M] output (-1 for padding)."""
    out = np.full(p.world * p.n_pad, -1, dtype=np.int64)
    for r in range(p.world):
        _, gc = local_tiles(tiles, p, r)
        out[r * p.n_pad:r * p.n_pad + len(gc)] = gc
    return out


class ShardedTWLayer:
    """One rank's share of a tile-wise sparse layer (CUDA)."""

    def __init__(self, W, tiles: TileSet, rank: int, world: int, dtype=None):
        import torch

        from .layer import TWLayer
        self.tiles, self.rank, self.world = tiles, rank, world
        self.plan = plan(tiles, world)
        self.local, self.global_cols = local_tiles(tiles, self.plan, rank)
        dtype = dtype or torch.float16
        idx = torch.from_numpy(self.global_cols.astype(np.int64)).to(W.device)
        W_local = W.index_select(1, idx).contiguous() if len(self.global_cols) else W[:, :1].contiguous()
        self.layer = TWLayer(self.local, dtype, W.device)
        self.layer.pack(W_local)
        self.order = column_order(tiles, self.plan)

    def masked_gemm(self, At, out=None):
        """Ct_local[n_pad, M]: this rank's kept columns (tile order), rows past n_local are zero."""
        import torch
        M = At.shape[1]
        if out is None:
            out = torch.zeros((self.plan.n_pad, M), dtype=At.dtype, device=At.device)
        n_loc = self.local.N
        self.layer.masked_gemm(At, out=out[:n_loc])
        return out

    def all_gather(self, Ct_local, out=None):
        """[world * n_pad, M]: every rank's slab, rank-major (`self.order` names the columns)."""
        import torch
        import torch.distributed as dist
        if out is None:
            out = torch.empty((self.world * self.plan.n_pad, Ct_local.shape[1]), dtype=Ct_local.dtype,
                              device=Ct_local.device)
        dist.all_gather_into_tensor(out, Ct_local.contiguous())
        return out

    # ------------------------------------------------------------------ fused GEMM + all-gather
    def make_gather_buffer(self, M: int, group=None):
        """Allocates the gathered output [world * n_pad, M] in peer-mapped (symmetric) memory and
        exchanges the mappings.  Collective: every rank of `group` must call it.  Returns
        (buffer, handle); keep both alive while the buffer is in use."""
        import torch
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm_mem
        group = group or dist.group.WORLD
        buf = symm_mem.empty((self.world * self.plan.n_pad, M), dtype=self.layer.dtype, device=self.layer.device)
        buf.zero_()
        handle = symm_mem.rendezvous(buf, group)
        torch.cuda.current_stream(self.layer.device).synchronize()
        handle.barrier()
        return buf, handle

    def masked_gemm_allgather(self, At, buf, handle, multicast: bool = False):
        """One kernel computes this rank's slab and stores every kept row into all ranks' gathered
        buffers (plain stores to peer-mapped memory: the transfer over NVLink overlaps the tiles still
        being computed).  The two barriers around it are device-side (signal pads of the symmetric
        allocation, enqueued on the current stream like the kernel, nothing blocks the host): peers
        must have finished with the buffer's previous contents before it is overwritten, and every
        rank's kernel, hence its stores, must have completed before anyone's stream goes on to read
        the buffer.  Consecutive steps therefore queue up back to back."""
        row0 = self.rank * self.plan.n_pad
        n_loc = self.local.N
        pitch = buf.stride(0) * buf.element_size()
        peers = [int(handle.buffer_ptrs[p]) + row0 * pitch for p in range(self.world) if p != self.rank]
        handle.barrier(channel=0)
        mc = int(getattr(handle, "multicast_ptr", 0) or 0) if multicast else 0
        if mc:
            # one multimem store per 16-byte piece: NVSwitch writes it into all ranks' buffers, so a GPU
            # sends its slab once instead of once per peer
            self.layer.masked_gemm(At, out=buf[row0:row0 + n_loc], multicast=mc + row0 * pitch)
        else:
            self.layer.masked_gemm(At, out=buf[row0:row0 + n_loc], peers=peers)
        handle.barrier(channel=1)
        return buf

    @staticmethod
    def has_multicast(handle) -> bool:
        """Whether the symmetric allocation has an NVSwitch multicast mapping."""
        return bool(int(getattr(handle, "multicast_ptr", 0) or 0))

    def assemble(self, gathered):
        """Full Ct[N, M] in the original column order (pruned columns zero).  A consumer that can
        take the permuted rows should use `self.order` instead of paying for this copy."""
        return assemble(gathered, self.order, self.tiles.N)

    def close(self):
        self.layer.close()


def assemble(gathered, order: np.ndarray, N: int):
    import torch
    valid = np.flatnonzero(order >= 0)
    out = torch.zeros((N, gathered.shape[1]), dtype=gathered.dtype, device=gathered.device)
    src = torch.from_numpy(valid.astype(np.int64)).to(gathered.device)
    dst = torch.from_numpy(order[valid].astype(np.int64)).to(gathered.device)
    out.index_copy_(0, dst, gathered.index_select(0, src))
    return out
