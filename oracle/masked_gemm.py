"""CPU oracle of the masked GEMM.  TEST INFRASTRUCTURE ONLY -- never imported by the product path.

Restates, in NumPy, what the reference defines the operation to be:

* the dense-masked form `matmul(x, kernel * mask)` of the reference's model code
  (Pruning/BERT/utils/modeling.py:992-1007; VGG/NMT rewire consumers to `w * mask`,
  Pruning/VGG/myhook.py:146-166);
* the compaction form its perf driver checks the kernel against: gather the kept K rows of A,
  multiply by the tile's compacted weights, scatter the result columns
  (Stream_Gemm_NN_reference, StreamMaskedGEMM/perf/basic_nn.cu:450-503; deleteRow/insertRow,
  :141-194; weight compaction gen_masked_stream_weight, :757-769);
* the driver's acceptance rule `checkout` (basic_nn.cu:771-798).

Parity status: the reference holds no stored vectors for GEMM results (its only check is the
in-binary comparison of the kernel with compaction + cuBLAS on unseeded random data,
basic_nn.cu:1081-1090), and its CUDA kernel cannot be run here (no GPU in the build container; the
Volta-only MMA bodies compile to nothing for sm_100).  The two restatements below are checked
against each other and against float64; beyond that the GEMM parity is unpinned by reference data.

Acceptance rules the GPU tests apply: `max_rel_error` (matrix level), `elementwise_violations`
(per element, relative with a floor) and the driver's own `checkout_errors` on data that does not
cancel (positive operands), where its absolute and ratio tests are both meaningful.
"""
from __future__ import annotations

import numpy as np


def masked_matmul_dense(A, W, mask, dtype=np.float32):
    """C[M, N] = A[M, K] @ (W[K, N] * mask)  (modeling.py:1001-1003, bias left out)."""
    A = np.asarray(A, dtype=dtype)
    Wm = np.asarray(W, dtype=dtype) * (np.asarray(mask) != 0)
    return A @ Wm


def pack_weights(W, tiles, rows_per_tile=128, ld=None, dtype=np.float32):
    """Wp[t*rows_per_tile + j, i] = W[kept_k_t[i], kept_n_t[j]]  (basic_nn.cu:757-769), zero padded."""
    W = np.asarray(W)
    kc = tiles.k_counts()
    if ld is None:
        ld = max(64, int(-(-int(kc.max(initial=0)) // 64) * 64))
    out = np.zeros((max(1, tiles.n_tiles) * rows_per_tile, ld), dtype=dtype)
    for t in range(tiles.n_tiles):
        r, c = tiles.tile_rows(t), tiles.tile_cols(t)
        if len(r) and len(c):
            out[t * rows_per_tile:t * rows_per_tile + len(c), :len(r)] = W[np.ix_(r, c)].T.astype(dtype)
    return out


def masked_matmul_compacted(At, W, tiles, alpha=1.0, beta=0.0, Ct=None, dtype=np.float32):
    """Ct[N, M] by compaction (basic_nn.cu:450-503): per tile, gather the kept rows of At[K, M],
    multiply by the compacted tile weights, write the kept columns' rows of Ct."""
    At = np.asarray(At, dtype=dtype)
    W = np.asarray(W, dtype=dtype)
    K, M = At.shape
    out = np.zeros((tiles.N, M), dtype=dtype) if Ct is None else np.array(Ct, dtype=dtype)
    for t in range(tiles.n_tiles):
        r, c = tiles.tile_rows(t), tiles.tile_cols(t)
        if len(c) == 0:
            continue
        acc = W[np.ix_(r, c)].T @ At[r, :] if len(r) else np.zeros((len(c), M), dtype=dtype)
        out[c, :] = alpha * acc + (beta * out[c, :] if beta != 0 else 0)
    return out


def checkout_errors(test, ref, err=1e-2):
    """Number of elements the reference's acceptance rule rejects (basic_nn.cu:785):
    v1/v2 > 1+err  or  v2/v1 > 1+err  or  |v2-v1| > err."""
    v2 = np.asarray(test, dtype=np.float32).ravel()
    v1 = np.asarray(ref, dtype=np.float32).ravel()
    with np.errstate(divide="ignore", invalid="ignore"):
        bad = (v1 / v2 > 1 + err) | (v2 / v1 > 1 + err) | (np.abs(v2 - v1) > err)
    return int(bad.sum())


def max_rel_error(test, ref):
    """max |test - ref| / max |ref|: the matrix-level relative error the acceptance bound uses."""
    test = np.asarray(test, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    denom = np.abs(ref).max()
    return float(np.abs(test - ref).max() / denom) if denom > 0 else float(np.abs(test).max())


def masked_matmul_rows(At, W, tiles, rows, dtype=np.float64):
    """Selected rows of Ct[N, M] by compaction (same definition as masked_matmul_compacted), for
    shapes whose full product is too slow for a test: row n of Ct is the kept rows of At weighted by
    column n of W restricted to the kept rows of the tile that owns n; zero when no tile keeps n."""
    At = np.asarray(At)
    W = np.asarray(W)
    out = np.zeros((len(rows), At.shape[1]), dtype=dtype)
    owner = np.full(tiles.N, -1, dtype=np.int64)
    for t in range(tiles.n_tiles):
        owner[tiles.tile_cols(t)] = t
    for i, n in enumerate(rows):
        t = owner[n]
        if t < 0:
            continue
        r = tiles.tile_rows(t)
        if len(r):
            out[i] = W[r, n].astype(dtype) @ At[r, :].astype(dtype)
    return out


def elementwise_violations(test, ref, rtol=1e-2, floor=1e-3):
    """Number of elements with |test - ref| > rtol * |ref| + floor * rms(ref): a per-element relative
    bound (the `max relative error <= 1e-2` of 16-bit outputs with fp32 accumulation) with an absolute
    floor tied to the typical magnitude, for elements that cancel to almost nothing."""
    test = np.asarray(test, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    rms = float(np.sqrt(np.mean(ref * ref))) if ref.size else 0.0
    return int((np.abs(test - ref) > rtol * np.abs(ref) + floor * rms).sum())


def im2col_nhwc(x, kh, kw):
    """The matrix a stride-1, same-padded kh x kw convolution multiplies with the kernel viewed as
    [(kh*kw*cin), cout] (img2col_forward, Pruning/VGG/prune_algo.py:16-24: row (r*kw + j)*cin + c):
    x is NHWC [B, H, W, C]; the result is [B*H*W, kh*kw*C] with pixels in (b, y, x) order."""
    x = np.asarray(x)
    B, H, W, C = x.shape
    ph, pw = (kh - 1) // 2, (kw - 1) // 2
    xp = np.zeros((B, H + kh - 1, W + kw - 1, C), dtype=x.dtype)
    xp[:, ph:ph + H, pw:pw + W, :] = x
    cols = [xp[:, r:r + H, j:j + W, :] for r in range(kh) for j in range(kw)]
    return np.concatenate(cols, axis=3).reshape(B * H * W, kh * kw * C)
