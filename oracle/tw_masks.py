"""CPU oracle of the tile-wise (TW / TEW) mask construction.  TEST INFRASTRUCTURE ONLY.

Restates the reference's mask algorithms in NumPy, one function per reference function, each citing
the lines it follows.  The arithmetic the reference delegates to NumPy (np.linalg.norm,
np.percentile; NumPy is not vendored and not version-pinned by the reference's environment.yml) is
kept as the same NumPy calls here, and separately spelled out as explicit IEEE-754 single steps in
`norm_rows_exact`, `norm_cols_exact` and `percentile_exact`, which is the specification the CUDA
kernels implement.  Parity is pinned to NumPy 2.3 (the version in the build image).

Pinning: tests/golden/*.npz hold masks produced by the reference's own prune_algo.py
(Pruning/VGG/prune_algo.py, imported unmodified by tests/golden/make_golden.py) on seeded inputs;
tests check every function below against them.  The BERT variants (Pruning/BERT/utils/MyHook.py,
pruning types 2, 7 and 8) are pinned the same way: make_golden.py imports that file unmodified beside
a stub `tensorflow` module and stores the masks its `granularity_pruning` and `pruning` produce.
`topk_l1` is a restatement only: no reference code performs that selection (parity unpinned).
"""
from __future__ import annotations

import numpy as np

# --------------------------------------------------------------------------------------------
# Column tilings
# --------------------------------------------------------------------------------------------


def fixed_bounds(N: int, G: int) -> np.ndarray:
    """Tiles of G columns, narrow last tile allowed (prune_algo.py:119-126)."""
    b = list(range(0, N, G)) + [N]
    return np.asarray(b, dtype=np.int64)


def regroup_bounds(col_mask, G: int) -> np.ndarray:
    """A tile ends right after its G-th kept column; no cut at the matrix edge (prune_algo.py:72-89)."""
    col_mask = np.asarray(col_mask).astype(bool)
    N = len(col_mask)
    bounds, count = [0], 0
    for c in range(N):
        if col_mask[c]:
            count += 1
        if count == G:
            if c + 1 < N:
                bounds.append(c + 1)
                count = 0
    bounds.append(N)
    return np.asarray(bounds, dtype=np.int64)


# --------------------------------------------------------------------------------------------
# Reference algorithms, restated
# --------------------------------------------------------------------------------------------


def _tile_row_norms(score, bounds, divide=True):
    """[n_tiles][K] L2 norm of every tile-row, divided by the tile width (prune_algo.py:128)."""
    out = []
    for t in range(len(bounds) - 1):
        w = score[:, bounds[t]:bounds[t + 1]]
        n = np.linalg.norm(w, axis=1)
        out.append(n / w.shape[1] if divide else n)
    return out


def _broadcast_rows(keep_per_tile, bounds, K):
    m = np.zeros((K, int(bounds[-1])), dtype=bool)
    for t, keep in enumerate(keep_per_tile):
        m[:, bounds[t]:bounds[t + 1]] = np.asarray(keep, dtype=bool)[:, None]
    return m


def tw1(scores, sparsity, granularity=128):
    """tiled_wise_1d (prune_algo.py:113-148): one global percentile over all tile-row norms of all
    layers in the group; keep strictly above it."""
    bounds = [fixed_bounds(s.shape[1], granularity) for s in scores]
    norms = [_tile_row_norms(s, b) for s, b in zip(scores, bounds)]
    flat = [v for layer in norms for tile in layer for v in tile]
    threshold = np.percentile(flat, sparsity)
    return [_broadcast_rows([n > threshold for n in layer], b, s.shape[0])
            for layer, b, s in zip(norms, bounds, scores)]


def tw2(scores, sparsity, granularity=128, remap=True, return_parts=False, col_sparsity=None):
    """tiled_wise_2d (prune_algo.py:55-111): column pruning by a global percentile of column norms
    (divided by K), regrouping of the surviving columns into tiles of `granularity`, then row
    pruning per tile by a second global percentile at the same (remapped) sparsity.
    col_sparsity (not in the reference, which ties both stages to one value at :61) gives the column
    stage a percentile of its own; the row stage then uses `sparsity` as passed."""
    if remap and col_sparsity is None:
        sparsity = 100 - np.sqrt(10000 - sparsity * 100)                      # :61
    col_norms = [np.linalg.norm(s, axis=0) / s.shape[0] for s in scores]       # :64
    threshold = np.percentile([v for n in col_norms for v in n],
                              sparsity if col_sparsity is None else col_sparsity)     # :65-66
    col_masks = [n > threshold for n in col_norms]                             # :67
    pruned = [np.tile(m, (s.shape[0], 1)).reshape(s.shape) * s for m, s in zip(col_masks, scores)]  # :68-69
    bounds = [regroup_bounds(m, granularity) for m in col_masks]               # :72-89
    norms = [_tile_row_norms(p, b) for p, b in zip(pruned, bounds)]            # :90
    flat = [v for layer in norms for tile in layer for v in tile]
    threshold2 = np.percentile(flat, sparsity)                                 # :93-95
    masks = [_broadcast_rows([n > threshold2 for n in layer], b, s.shape[0]) * cm[None, :]
             for layer, b, s, cm in zip(norms, bounds, scores, col_masks)]     # :99-109
    if return_parts:
        return masks, col_masks, bounds
    return masks


def tw_mix(scores, g1percent, layer_masks):
    """tw_mix_fn (prune_algo.py:151-177): element-wise residual on top of a tile-wise mask.  Every
    element's magnitude (norm of a 1-element vector) minus its TW mask bit is ranked globally; the
    top g1percent percent are added to the mask."""
    vals = []
    for s, m in zip(scores, layer_masks):
        cols = [np.linalg.norm(s[:, n:n + 1], axis=1) / 1 for n in range(s.shape[1])]   # :156-157
        vals.append(np.asarray(cols) - np.asarray(m).transpose())                        # :159 -> [N, K]
    threshold = np.percentile([v for layer in vals for row in layer for v in row], 100 - g1percent)  # :165-166
    out = []
    for v, m in zip(vals, layer_masks):
        mask1 = (v > threshold).transpose()                                              # :171-173
        out.append(np.asarray(m, dtype=bool) + mask1)                                    # :175
    return out


def tw1m(scores, sparsity, granularity=128, g1percent=5):
    """tiled_wise_1d_mix (prune_algo.py:180-184)."""
    return tw_mix(scores, g1percent, tw1(scores, sparsity + g1percent, granularity))


def tw2m(scores, sparsity, granularity=128, g1percent=1):
    """tiled_wise_2d_mix (prune_algo.py:187-191)."""
    return tw_mix(scores, g1percent, tw2(scores, sparsity + g1percent, granularity))


def bert_type7(scores, sparsity, granularity=128):
    """BERT pruning type 7 (Pruning/BERT/utils/MyHook.py:226-258): tw1 with divisibility required."""
    for s in scores:
        if s.shape[1] % granularity != 0:
            raise ValueError("type 7 needs N divisible by the granularity (MyHook.py:222-224)")
    return tw1(scores, sparsity, granularity)


def bert_type8(scores, sparsity, granularity=128):
    """BERT pruning type 8 (MyHook.py:260-313): tw2 without the sparsity remap."""
    return tw2(scores, sparsity, granularity, remap=False)


def tw_cols_rows(scores, col_sparsity, row_sparsity, granularity=128):
    """The machinery of tiled_wise_2d with independent column and row percentiles ("10 % of the
    columns, then 75 % of the rows of every tile").  No reference function has this call shape."""
    return tw2(scores, row_sparsity, granularity, remap=False, col_sparsity=col_sparsity)


def bert_type2(score, sparsity, granularity=128):
    """granularity_pruning (MyHook.py:202-214): per-tile percentile of un-normalised L2 row norms."""
    K, N = score.shape
    if N % granularity != 0:
        raise ValueError("granularity_pruning needs N divisible by the granularity")
    bounds = fixed_bounds(N, granularity)
    keep = []
    for n in _tile_row_norms(score, bounds, divide=False):
        keep.append(n > np.percentile(n, sparsity))
    return _broadcast_rows(keep, bounds, K)


def topk_l1(score, sparsity, granularity=128):
    """Per-tile top-k by L1 row magnitude, ties to the lower row index (no reference code does this;
    it is the selection rule of the benchmark specification).  k = round(K * (1 - sparsity/100)).
    The L1 sums are accumulated left to right in float32."""
    score = np.asarray(score, dtype=np.float32)
    K, N = score.shape
    bounds = fixed_bounds(N, granularity)
    k_keep = int(round(K * (1.0 - float(sparsity) / 100.0)))
    keep = []
    for t in range(len(bounds) - 1):
        a = np.abs(score[:, bounds[t]:bounds[t + 1]])
        l1 = np.zeros(K, dtype=np.float32)
        for c in range(a.shape[1]):
            l1 = (l1 + a[:, c]).astype(np.float32)
        order = np.argsort(-l1.astype(np.float64), kind="stable")       # descending, ties -> lower index
        kt = np.zeros(K, dtype=bool)
        kt[order[:k_keep]] = True
        keep.append(kt)
    return _broadcast_rows(keep, bounds, K)


def ew(scores, sparsity):
    """Element-wise baseline (prune_algo.py:38-53): one percentile over |score| of all layers.  The
    reference flattens through Python lists, so the percentile runs on float64 copies of the float32
    values and the threshold is a float64; `abs(layer) > threshold` compares exactly."""
    flat = np.concatenate([np.abs(np.asarray(l)).reshape(-1).astype(np.float64) for l in scores])
    thr = percentile_f64(flat, float(sparsity))
    return [np.abs(np.asarray(l)) > thr for l in scores]


def vw(scores, sparsity):
    """Vector-wise baseline (prune_algo.py:196-227): along K, in blocks of 16 rows of one column,
    keep what exceeds the block's (topk+1)-th largest value, topk = int((1 - sparsity/100) * 16); a
    block no longer than topk+1 keeps what exceeds 0.  Returns float64 0/1 arrays like the reference."""
    block = 16
    topk = int((1 - sparsity / 100) * block)
    out = []
    for layer in scores:
        sc = np.asarray(layer)
        K, N = sc.shape
        mask = np.zeros((K, N))
        for k0 in range(0, K, block):
            blk = sc[k0:k0 + block]                              # [len, N]
            if topk + 1 < blk.shape[0]:
                thr = np.sort(blk, axis=0)[-(topk + 1)]          # per column
            else:
                thr = np.zeros(N, dtype=sc.dtype)
            mask[k0:k0 + block] = blk > thr[None, :]
        out.append(mask)
    return out


def percentile_f64(values, q):
    """np.percentile(float64 array, Python float q), method 'linear', step by step in double."""
    v = np.sort(np.asarray(values, dtype=np.float64))
    n = len(v)
    virt = np.float64(n - 1) * (np.float64(q) / np.float64(100))
    prev = np.floor(virt)
    gamma = np.float64(virt - prev)
    pi, ni = int(prev), int(prev) + 1
    if virt >= n - 1:
        pi = ni = n - 1
    a, b = v[pi], v[ni]
    diff = np.float64(b - a)
    if gamma >= 0.5:
        return np.float64(b - diff * (np.float64(1) - gamma))
    return np.float64(a + diff * gamma)


def bw(scores, sparsity, granularity=32, return_norms=False):
    """Block-wise baseline (prune_algo.py:229-264): Frobenius norm of every granularity x granularity
    block, one percentile over the blocks of all layers, blocks above it kept.  The norm of a 2-D slice
    goes through BLAS sdot, so its last bits depend on the host CPU; `return_norms` also returns the
    block norms in float64 and the threshold, with which a test can tell the blocks that sit within
    rounding distance of the threshold."""
    norms, exact = [], []
    for s in scores:
        for i in range(0, s.shape[0], granularity):
            for j in range(0, s.shape[1], granularity):
                blk = s[i:i + granularity, j:j + granularity]
                norms.append(np.linalg.norm(blk))
                exact.append(np.sqrt(np.sum(blk.astype(np.float64) ** 2)))
    threshold = np.percentile(norms, sparsity)
    block_mask = norms > threshold
    out, idx = [], 0
    for s in scores:
        mask = np.zeros(s.shape)
        for i in range(0, s.shape[0], granularity):
            for j in range(0, s.shape[1], granularity):
                if block_mask[idx]:
                    mask[i:i + granularity, j:j + granularity] = 1
                idx += 1
        out.append(mask)
    if return_norms:
        return out, np.asarray(exact), float(threshold)
    return out


ALGOS = {"tw1": tw1, "tw2": tw2, "tw1m": tw1m, "tw2m": tw2m, "ew": ew, "vw": vw, "bw": bw}


def pruning_fun(name):
    """Same dispatch as the reference (prune_algo.py:267-278)."""
    return ALGOS[name]


# --------------------------------------------------------------------------------------------
# The NumPy arithmetic, spelled out (specification of the CUDA kernels)
# --------------------------------------------------------------------------------------------

_f32 = np.float32


def pairwise_sum_exact(a):
    """NumPy's float32 add.reduce over a contiguous run (verified bit for bit against
    np.add.reduce for lengths 1..1280): fewer than 8 elements are added left to right; up to 128
    use eight running sums over elements j, j+8, j+16, ... combined as
    ((r0+r1)+(r2+r3))+((r4+r5)+(r6+r7)) followed by the <8 leftover elements in order; longer runs
    split at n//2 rounded down to a multiple of 8 and add the two halves' sums."""
    a = np.asarray(a, dtype=_f32)
    n = len(a)
    if n < 8:
        r = _f32(0.0)
        for x in a:
            r = _f32(r + x)
        return r
    if n <= 128:
        r = [a[j] for j in range(8)]
        i = 8
        while i < n - (n % 8):
            for j in range(8):
                r[j] = _f32(r[j] + a[i + j])
            i += 8
        res = _f32(_f32(_f32(r[0] + r[1]) + _f32(r[2] + r[3])) + _f32(_f32(r[4] + r[5]) + _f32(r[6] + r[7])))
        while i < n:
            res = _f32(res + a[i])
            i += 1
        return res
    n2 = n // 2
    n2 -= n2 % 8
    return _f32(pairwise_sum_exact(a[:n2]) + pairwise_sum_exact(a[n2:]))


def norm_rows_exact(x):
    """np.linalg.norm(x, axis=1) for float32 x: squares rounded to float32, pairwise sum, sqrt."""
    x = np.asarray(x, dtype=_f32)
    sq = (x * x).astype(_f32)
    return np.asarray([np.sqrt(pairwise_sum_exact(r)) for r in sq], dtype=_f32)


def norm_cols_exact(x):
    """np.linalg.norm(x, axis=0) for C-ordered float32 x: squares, summed down the rows in order."""
    x = np.asarray(x, dtype=_f32)
    sq = (x * x).astype(_f32)
    acc = sq[0].copy()
    for k in range(1, x.shape[0]):
        acc = (acc + sq[k]).astype(_f32)
    return np.sqrt(acc)


def percentile_exact(values, q):
    """np.percentile(list of float32, q), method 'linear', step by step.

    The arithmetic type follows q: a Python number is "weak" and everything stays float32
    (q/100, the virtual index (n-1)*q and the interpolation are single-precision operations); a
    NumPy float64 scalar (what tw2's `100 - np.sqrt(...)` produces) makes them double precision and
    the result a float64.  Returns (threshold, prev_index, next_index)."""
    v = np.sort(np.asarray(values, dtype=_f32))
    n = len(v)
    wide = isinstance(q, np.floating) and not isinstance(q, np.float32)
    T = np.float64 if wide else _f32
    qf = T(q) / T(100)
    virt = T(n - 1) * qf
    prev = np.floor(virt)
    gamma = T(virt - prev)
    pi, ni = int(prev), int(prev) + 1
    if virt >= n - 1:
        pi = ni = n - 1
    a, b = T(v[pi]), T(v[ni])
    diff = T(_f32(v[ni] - v[pi]))        # b - a is a float32 operation in both paths (array elements)
    if gamma >= T(0.5):
        res = T(b - T(diff * T(T(1) - gamma)))
    else:
        res = T(a + T(diff * gamma))
    return res, pi, ni
