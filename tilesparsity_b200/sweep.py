"""Sweep of the benchmark configurations: masked GEMM vs cuBLAS dense on one B200.

    python -m tilesparsity_b200.sweep [--configs bert,vgg,lstm,square,balance,masks] [--iters 200]

For every configuration the masks are built on the GPU from seeded synthetic weights (the reference's
algorithms, tilesparsity_b200.masks), the layer is packed, and the tensor-core masked GEMM is timed
from a CUDA graph next to `torch.matmul` (cuBLAS) on the same dense shapes, with activations and
outputs rotating over enough buffers to exceed L2.  One JSON line per row.  Shapes and
distributions stand in for the reference's models (BERT-base, VGG16 conv5, NMT LSTM), which are not
available here.
"""
from __future__ import annotations

import argparse
import json

import numpy as np
import torch

from . import synth
from .layer import TEWLayer, TWLayer
from .masks import build_mask
from .tiles import tiles_from_lists

L2_BYTES = 126 << 20


def _time_graph(fn, n_sets: int, iters: int) -> float:
    """Microseconds per call of fn(i), i cycling over n_sets buffer sets, replayed from a CUDA graph."""
    for i in range(n_sets):
        fn(i)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for i in range(n_sets):
            fn(i)
    g.replay()
    torch.cuda.synchronize()
    reps = max(1, iters // n_sets)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        g.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / (reps * n_sets)


def run_case(name, M, K, N, dtype, layer_fn, iters, note=""):
    dev = torch.device("cuda", torch.cuda.current_device())
    gen = torch.Generator(device=dev).manual_seed(hash(name) % (2 ** 31))
    W = torch.randn((K, N), generator=gen, device=dev, dtype=torch.float32) * 0.02
    layer, kept_flops_per_row, extra = layer_fn(W)
    per_set = (K * M + N * M) * 2
    n_sets = int(max(2, min(8, (2 * L2_BYTES) // per_set + 1)))
    At = [torch.randn((K, M), generator=gen, device=dev, dtype=torch.float32).to(dtype) for _ in range(n_sets)]
    Ct = [torch.zeros((N, M), dtype=dtype, device=dev) for _ in range(n_sets)]
    Wt = W.t().contiguous().to(dtype)
    t_m = _time_graph(lambda i: layer.masked_gemm(At[i], out=Ct[i]), n_sets, iters)
    t_d = _time_graph(lambda i: torch.matmul(Wt, At[i], out=Ct[i]), n_sets, iters)
    kept = kept_flops_per_row * M
    row = {"config": name, "M": M, "K": K, "N": N, "dtype": str(dtype).split(".")[-1], "masked_us": round(t_m, 2),
           "cublas_dense_us": round(t_d, 2), "speedup_vs_cublas_dense": round(t_d / t_m, 3),
           "kept_tflops": round(kept / t_m / 1e6, 1), "dense_tflops": round(2.0 * M * K * N / t_d / 1e6, 1),
           "kept_fraction": round(kept / (2.0 * M * K * N), 4), "buffer_sets": n_sets, "note": note, **extra}
    print(json.dumps(row), flush=True)
    layer.close()
    return row


def tw_layer(sparsity, dtype, algo="tw1"):
    def fn(W):
        res = build_mask(algo, [W.abs()], sparsity, 128)
        layer = TWLayer(res.tiles[0], dtype, W.device)
        layer.pack(W)
        return layer, res.tiles[0].kept_flops_per_row(), {"tiles": res.tiles[0].n_tiles}
    return fn


def col_then_row_layer(col_sparsity, row_sparsity, dtype):
    """Column pruning and tile-wise row pruning with independent sparsities (the reference's tw2 ties
    both to one remapped value, Pruning/VGG/prune_algo.py:61): columns by L2 norm, survivors regrouped
    into tiles of 128, rows per tile by a global percentile of the tile-row norms."""
    def fn(W):
        K, N = W.shape
        cn = W.norm(dim=0)
        keep_cols = cn > torch.quantile(cn, col_sparsity / 100.0)
        cols = torch.nonzero(keep_cols).flatten()
        groups = list(torch.split(cols, 128))
        norms = torch.stack([W[:, g].norm(dim=1) / len(g) for g in groups])          # [tiles, K]
        thr = torch.quantile(norms.flatten(), row_sparsity / 100.0)
        lists = [torch.nonzero(norms[t] > thr).flatten().cpu().numpy().astype(np.int32) for t in range(len(groups))]
        ts = tiles_from_lists(K, N, 128, lists, col_mask=keep_cols.cpu().numpy())
        layer = TWLayer(ts, dtype, W.device)
        layer.pack(W)
        return layer, ts.kept_flops_per_row(), {"tiles": ts.n_tiles}
    return fn


def run_mask_case(algo, K, N, sparsity, g1=None, reps=5):
    """Wall-clock of the host-synchronous mask build (scores resident on the GPU) and its HBM-level
    bytes: the scores read once per norm pass plus the dense 0/1 mask written."""
    import time
    dev = torch.device("cuda", torch.cuda.current_device())
    gen = torch.Generator(device=dev).manual_seed(K * 31 + N)
    W = (torch.randn((K, N), generator=gen, device=dev, dtype=torch.float32) * 0.02).abs()
    build_mask(algo, [W], sparsity, 128, g1)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(reps):
        res = build_mask(algo, [W], sparsity, 128, g1)
    torch.cuda.synchronize()
    dt = (time.perf_counter() - t0) / reps
    passes = {"tw1": 1, "tw2": 2, "tw1m": 2, "tw2m": 3}[algo]
    nbytes = K * N * (4 * passes + 1)
    row = {"config": f"mask_{algo}_{K}x{N}", "K": K, "N": N, "sparsity": sparsity, "seconds": round(dt, 6),
           "bytes": nbytes, "gbs": round(nbytes / dt / 1e9, 1), "density": round(float(res.masks[0].float().mean()), 4)}
    print(json.dumps(row), flush=True)
    return row


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--configs", default="bert,vgg,lstm,square")
    ap.add_argument("--iters", type=int, default=200)
    ap.add_argument("--sizes", default="4096,8192,16384")
    a = ap.parse_args(argv)
    want = set(a.configs.split(","))
    rows = []
    if "masks" in want:
        for algo, K, N, sp, g1 in [("tw1", 768, 3072, 75.0, None), ("tw1", 2048, 4096, 75.0, None),
                                    ("tw1", 8192, 8192, 75.0, None), ("tw2", 4608, 512, 75.0, None),
                                    ("tw2", 8192, 8192, 75.0, None), ("tw1m", 2048, 4096, 75.0, 1.5)]:
            rows.append(run_mask_case(algo, K, N, sp, g1))
    if "bert" in want:
        for sp in (50.0, 75.0, 90.0):
            for nm, (K, N) in synth.BERT_BASE_LAYER.items():
                rows.append(run_case(f"bert_{nm}_tw{int(sp)}", 4096, K, N, torch.float16, tw_layer(sp, torch.float16), a.iters))
    if "vgg" in want:
        # conv5 as a GEMM over the im2col matrix: the reference's tw2 at 75 % (both stages at the
        # remapped 50 %), and 10 % column pruning followed by 75 % tile-wise row pruning.
        rows.append(run_case("vgg16_conv5_tw2_75", 12544, 4608, 512, torch.bfloat16, tw_layer(75.0, torch.bfloat16, "tw2"),
                             a.iters, "tw2 at 75 %: 50 % of columns x 50 % of rows per tile"))
        rows.append(run_case("vgg16_conv5_c10_k75", 12544, 4608, 512, torch.bfloat16,
                             col_then_row_layer(10.0, 75.0, torch.bfloat16), a.iters,
                             "10 % of columns pruned, then 75 % of the rows of every tile"))
    if "balance" in want:
        # per-tile percentile (BERT type 2, equal kept-K per tile) next to the global percentile of tw1
        for nm in ("ffn1", "ffn2"):
            K, N = synth.BERT_BASE_LAYER[nm]
            rows.append(run_case(f"bert_{nm}_type2_75", 4096, K, N, torch.float16,
                                 tw_layer(75.0, torch.float16, "bert_type2"), a.iters, "equal kept-K per tile"))
            rows.append(run_case(f"bert_{nm}_tw1_75", 4096, K, N, torch.float16, tw_layer(75.0, torch.float16), a.iters,
                                 "global percentile: kept-K varies per tile"))
    if "lstm" in want:
        def tew(W):
            res = build_mask("tw1m", [W.abs()], 75.0, 128, 1.5, want_residual=True)
            layer = TEWLayer(W, res.tiles[0], res.residuals[0], torch.float16)
            return layer, res.tiles[0].kept_flops_per_row() + 2 * layer.nnz, {"residual_nnz": layer.nnz}
        rows.append(run_case("nmt_lstm_tew_75_1.5", 6400, 2048, 4096, torch.float16, tew, a.iters))
        rows.append(run_case("nmt_lstm_tw1_75", 6400, 2048, 4096, torch.float16, tw_layer(75.0, torch.float16), a.iters))
    if "square" in want:
        for n in [int(x) for x in a.sizes.split(",")]:
            def sq(W, n=n):
                nt = (n + 127) // 128
                counts = synth.beta_skewed_counts(n, nt, 0.25, 5000 + int(np.log2(n)))
                g = synth.rng(5000 + int(np.log2(n)))
                lists = [np.sort(g.choice(n, size=int(c), replace=False)).astype(np.int32) for c in counts]
                ts = tiles_from_lists(n, n, 128, lists)
                layer = TWLayer(ts, torch.bfloat16, W.device)
                layer.pack(W)
                return layer, ts.kept_flops_per_row(), {"tiles": nt, "kept_k_min": int(counts.min()), "kept_k_max": int(counts.max())}
            rows.append(run_case(f"square_{n}_beta25", n, n, n, torch.bfloat16, sq, max(20, a.iters // 4)))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
