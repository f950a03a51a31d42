"""Host-side tile bookkeeping: 0/1 masks <-> per-tile index lists.

This is the glue the reference leaves to its driver and export hook: the column-tile partition
(StreamMaskedGEMM/perf/basic_nn.cu:836-885), the "index minus position" offset lists
(mask_gen, basic_nn.cu:697-718; convert_mask_to_offset, Pruning/BERT/utils/MyHook.py:66-74) and the
regrouping of surviving columns into tiles of G kept columns (Pruning/VGG/prune_algo.py:72-89).
Pure NumPy integer work on small arrays; the heavy lifting (packing, GEMM, mask scoring) is CUDA.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np


@dataclass
class TileSet:
    """CSR description of a tile-wise sparse [K, N] weight matrix.

    tile_bounds[t] .. tile_bounds[t+1] is the column range of tile t in the dense matrix;
    kept_k[tile_k_ptr[t]:tile_k_ptr[t+1]] are its kept rows (ascending, absolute);
    kept_n[tile_n_ptr[t]:tile_n_ptr[t+1]] are its kept columns (ascending, absolute).
    """

    K: int
    N: int
    G: int
    tile_bounds: np.ndarray
    tile_k_ptr: np.ndarray
    kept_k: np.ndarray
    tile_n_ptr: np.ndarray
    kept_n: np.ndarray

    @property
    def n_tiles(self) -> int:
        return len(self.tile_k_ptr) - 1

    def k_counts(self) -> np.ndarray:
        return np.diff(self.tile_k_ptr)

    def n_counts(self) -> np.ndarray:
        return np.diff(self.tile_n_ptr)

    def tile_rows(self, t: int) -> np.ndarray:
        return self.kept_k[self.tile_k_ptr[t]:self.tile_k_ptr[t + 1]]

    def tile_cols(self, t: int) -> np.ndarray:
        return self.kept_n[self.tile_n_ptr[t]:self.tile_n_ptr[t + 1]]

    def lists(self) -> list:
        """Per-tile kept-row lists."""
        return [self.tile_rows(t) for t in range(self.n_tiles)]

    def col_mask(self) -> np.ndarray:
        m = np.zeros(self.N, dtype=bool)
        m[self.kept_n] = True
        return m

    def kept_flops_per_row(self) -> int:
        return int(2 * np.sum(self.k_counts().astype(np.int64) * self.n_counts().astype(np.int64)))

    def dense_mask(self) -> np.ndarray:
        """The 0/1 mask [K, N] these tiles describe."""
        m = np.zeros((self.K, self.N), dtype=bool)
        for t in range(self.n_tiles):
            r, c = self.tile_rows(t), self.tile_cols(t)
            if len(r) and len(c):
                m[np.ix_(r, c)] = True
        return m

    def relative_k(self) -> np.ndarray:
        """Kept rows in the reference's offset format: index minus position inside the tile."""
        out = self.kept_k.copy()
        for t in range(self.n_tiles):
            a, b = self.tile_k_ptr[t], self.tile_k_ptr[t + 1]
            out[a:b] -= np.arange(b - a, dtype=out.dtype)
        return out

    def relative_n(self, tile_local: bool = True) -> np.ndarray:
        """Kept columns as offsets; tile_local subtracts the tile's first column as the reference's
        per-tile C base pointer does (off_C, basic_nn.cu:875-885)."""
        out = self.kept_n.copy()
        for t in range(self.n_tiles):
            a, b = self.tile_n_ptr[t], self.tile_n_ptr[t + 1]
            out[a:b] -= np.arange(b - a, dtype=out.dtype)
            if tile_local:
                out[a:b] -= self.tile_bounds[t]
        return out


def mask_to_offsets(mask_1d) -> np.ndarray:
    """0/1 vector -> ascending kept indices minus their position (MyHook.py:66-74)."""
    idx = np.flatnonzero(np.asarray(mask_1d) != 0).astype(np.int32)
    return idx - np.arange(len(idx), dtype=np.int32)


def offsets_to_indices(offsets) -> np.ndarray:
    offsets = np.asarray(offsets, dtype=np.int32)
    return offsets + np.arange(len(offsets), dtype=np.int32)


def tile_bounds_from_col_mask(col_mask, G: int) -> np.ndarray:
    """Column split points: a tile ends right after its G-th kept column (prune_algo.py:72-89).

    Trailing pruned columns fall into the next tile; a cut that would land on the matrix edge is not
    made, so the last tile may hold fewer than G kept columns (or none).  With every column kept
    this is the fixed partition into tiles of G columns, narrow last tile allowed
    (prune_algo.py:119-126).
    """
    col_mask = np.asarray(col_mask).astype(bool)
    N = len(col_mask)
    bounds = [0]
    count = 0
    for c in range(N):
        if col_mask[c]:
            count += 1
        if count == G:
            if c + 1 < N:
                bounds.append(c + 1)
                count = 0
    bounds.append(N)
    return np.asarray(bounds, dtype=np.int32)


def tiles_from_lists(K: int, N: int, G: int, kept_k_lists, col_mask=None) -> TileSet:
    """Per-tile kept-row lists + a global column mask -> TileSet."""
    if col_mask is None:
        col_mask = np.ones(N, dtype=bool)
    col_mask = np.asarray(col_mask).astype(bool)
    if col_mask.shape != (N,):
        raise ValueError(f"col_mask must have shape ({N},)")
    bounds = tile_bounds_from_col_mask(col_mask, G)
    n_tiles = len(bounds) - 1
    if len(kept_k_lists) != n_tiles:
        raise ValueError(f"expected {n_tiles} kept-row lists, got {len(kept_k_lists)}")
    kp, npz, kk, nn = [0], [0], [], []
    for t in range(n_tiles):
        rows = np.asarray(kept_k_lists[t], dtype=np.int32).reshape(-1)
        if len(rows) and (rows.min() < 0 or rows.max() >= K or np.any(np.diff(rows) <= 0)):
            raise ValueError(f"tile {t}: kept rows must be strictly ascending in [0, {K})")
        cols = (bounds[t] + np.flatnonzero(col_mask[bounds[t]:bounds[t + 1]])).astype(np.int32)
        kk.append(rows)
        nn.append(cols)
        kp.append(kp[-1] + len(rows))
        npz.append(npz[-1] + len(cols))
    cat = lambda xs: np.concatenate(xs).astype(np.int32) if xs else np.zeros(0, np.int32)
    return TileSet(K, N, G, bounds, np.asarray(kp, np.int32), cat(kk), np.asarray(npz, np.int32), cat(nn))


def tiles_from_mask(mask, G: int, col_mask=None, strict: bool = True) -> TileSet:
    """0/1 mask [K, N] with tile-wise structure -> TileSet.

    col_mask None means "no column was pruned" (tw1: fixed tiles of G columns).  For masks built
    with column pruning (tw2) pass the column mask so the tile boundaries follow the regrouping
    rule.  With strict=True a mask that is not purely tile-wise (e.g. a TEW mask with residual
    elements) raises; with strict=False the row set of a tile is the rows kept in its first kept
    column intersected over all kept columns (the TW part), and the caller handles the rest.
    """
    mask = np.asarray(mask) != 0
    K, N = mask.shape
    if col_mask is None:
        col_mask = np.ones(N, dtype=bool)
    col_mask = np.asarray(col_mask).astype(bool)
    bounds = tile_bounds_from_col_mask(col_mask, G)
    lists = []
    for t in range(len(bounds) - 1):
        cols = bounds[t] + np.flatnonzero(col_mask[bounds[t]:bounds[t + 1]])
        if len(cols) == 0:
            lists.append(np.zeros(0, np.int32))
            continue
        sub = mask[:, cols]
        rows_all = sub.all(axis=1)
        if strict and not np.array_equal(rows_all, sub.any(axis=1)):
            raise ValueError(f"tile {t} is not tile-wise: its kept columns keep different rows")
        lists.append(np.flatnonzero(rows_all).astype(np.int32))
    ts = tiles_from_lists(K, N, G, lists, col_mask)
    if strict and not np.array_equal(ts.dense_mask(), mask):
        raise ValueError("mask keeps elements outside its tiles' kept rows x kept columns")
    return ts


def reference_partition(N: int, N_pruned: int, G: int = 128):
    """The perf driver's tile partition (basic_nn.cu:836-861): block_num = ceil(N_pruned / G) tiles;
    each owns N // block_num dense columns and computes G of them, the last takes the remainders.
    Returns (N_ori, N_cal) as int lists."""
    block_num = (N_pruned + G - 1) // G
    n_ori, n_cal = [], []
    for _ in range(block_num - 1):
        n_ori.append(N // block_num)
        n_cal.append(G)
    if block_num > 0:
        n_ori.append(N - sum(n_ori))
        n_cal.append(N_pruned - sum(n_cal))
    return n_ori, n_cal
