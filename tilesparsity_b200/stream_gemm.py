"""The perf driver `test_basic_nn <M> <N> <K> <N_pruned> <K_pruned>` and `Stream_Gemm_NN`.

Mirrors the reference driver (StreamMaskedGEMM/perf/basic_nn.cu): same positional arguments, same
rounding of every size up to a multiple of 8 (:1152-1158), same tile partition (:836-885), random
sorted index subsets per tile stored as relative offsets (mask_gen, :697-741), weights compacted
column-major with ldb = K (gen_masked_stream_weight, :757-769), alpha = 1, beta = 0, mean of 100
iterations, and the same output lines: `CUTLASS GEMM : %f us.` twice (the dense baseline on
zero-filled weights; cuBLAS here, where the reference ran CUTLASS 1.3), `Stream  GEMM : %f us.`
once, then PASSED / incorrect lines on stderr for the driver's cross-checks (:1081-1090): the masked
kernel against compaction + cuBLAS per tile, against the CUDA-core twin, and against the dense
product on zero-filled weights.  Every GEMM runs on the GPU; this module never computes on the CPU.

    python -m tilesparsity_b200.stream_gemm 12800 768 768 384 384
    python -m tilesparsity_b200.stream_gemm 4096 3072 768 --sparsity 75 --G 128   # TW-K only
"""
from __future__ import annotations

import argparse
import ctypes as C
import sys

import numpy as np
import torch

from . import _lib
from ._lib import check, lib
from .tiles import reference_partition

N_DIM = 128          # columns computed per tile (basic_nn.cu:73)
MAX_BLOCK_NUM = 32   # tiles per call (basic_nn.cu:74)


def mask_gen(rng: np.random.Generator, n: int, n_pruned: int) -> np.ndarray:
    """Sorted random subset of n_pruned out of n, as relative offsets (basic_nn.cu:697-718)."""
    keep = np.sort(rng.permutation(n)[:n_pruned]).astype(np.int32)
    return keep - np.arange(n_pruned, dtype=np.int32)


def prepare_stream_gemm_nn(M: int, N: int, K: int, alpha: float, A: torch.Tensor, B: torch.Tensor, beta: float,
                           C_out: torch.Tensor, block_num: int, N_cal, K_cal, mask_n, mask_k, off_B, off_C):
    """Marshals the arguments of Stream_Gemm_NN once and returns a zero-argument callable that issues
    the call (a C caller passes its arrays directly; from Python the conversion of six arrays per call
    would cost more than the GEMM)."""
    dt = _lib.TS_DTYPE_BF16 if A.dtype == torch.bfloat16 else _lib.TS_DTYPE_F16
    IntArr = C.c_int * block_num
    PtrArr = C.c_void_p * block_num
    args = (M, N, K, alpha, C.c_void_p(A.data_ptr()), C.c_void_p(B.data_ptr()), beta, C.c_void_p(C_out.data_ptr()),
            block_num, IntArr(*[int(v) for v in N_cal]), IntArr(*[int(v) for v in K_cal]),
            PtrArr(*[t.data_ptr() for t in mask_n]), PtrArr(*[t.data_ptr() for t in mask_k]),
            IntArr(*[int(v) for v in off_B]), IntArr(*[int(v) for v in off_C]), dt)
    keep_alive = (A, B, C_out, list(mask_n), list(mask_k))
    device = A.device

    def call() -> None:
        _ = keep_alive
        check(lib.ts_stream_gemm_nn(*args, C.c_void_p(torch.cuda.current_stream(device).cuda_stream)))

    return call


def stream_gemm_nn(M: int, N: int, K: int, alpha: float, A: torch.Tensor, B: torch.Tensor, beta: float,
                   C_out: torch.Tensor, block_num: int, N_cal, K_cal, mask_n, mask_k, off_B, off_C) -> None:
    """Stream_Gemm_NN with the reference's argument list (basic_nn.cu:378-393).

    A: [K, M] (column-major M x K); B: the compacted tiles, column-major with ldb = K; C_out: [N, M];
    mask_n / mask_k: lists of int32 CUDA tensors holding relative offsets; the other arrays are host
    integer sequences.  One launch on the current stream, no synchronisation.
    """
    with torch.cuda.device(A.device):
        prepare_stream_gemm_nn(M, N, K, alpha, A, B, beta, C_out, block_num, N_cal, K_cal, mask_n, mask_k,
                               off_B, off_C)()


def checkout(test: torch.Tensor, ref: torch.Tensor, err: float, out=sys.stderr) -> int:
    """The driver's comparison (basic_nn.cu:771-798), evaluated on the GPU; returns the error count.

    The reference flags v1/v2 > 1+err, v2/v1 > 1+err or |v2-v1| > err.  Its ratio tests only ever
    compared bit-identical code paths; between independent summation orders they misfire on results
    that cancel to almost zero, so here they apply where either magnitude reaches err (below that
    the absolute test is the only one that can mean anything).
    """
    errors = checkout_counts(test, ref, err)[0]
    if errors > 0:
        print(f"CUTLASS results incorrect. Errors : {errors} / {test.numel()}\n", file=out)
    else:
        print("PASSED !!!\n", file=out)
    return errors


def checkout_counts(test: torch.Tensor, ref: torch.Tensor, err: float):
    """(errors under the rule `checkout` applies, errors under the reference's rule to the letter).

    The second count includes the elements whose magnitudes are below err on both sides and whose
    ratio alone trips the reference's test; the difference between the two is what the magnitude
    guard lets through."""
    v2, v1 = test.float(), ref.float()
    ratio = (v1 / v2 > 1 + err) | (v2 / v1 > 1 + err)
    far = (v2 - v1).abs() > err
    big = (v1.abs() >= err) | (v2.abs() >= err)
    return int(((big & ratio) | far).sum().item()), int((ratio | far).sum().item())


def _time_us(fn, iters: int) -> float:
    fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / iters


def run(M: int, N: int, K: int, N_pruned: int, K_pruned: int, dtype=torch.float16, iters: int = 100, seed: int = 0,
        check_results: bool = True, err: float = 1e-2, out=sys.stdout) -> dict:
    if not torch.cuda.is_available():
        raise RuntimeError("test_basic_nn needs a CUDA device")
    M, N, K, N_pruned, K_pruned = [(v + 7) // 8 * 8 for v in (M, N, K, N_pruned, K_pruned)]
    if not (0 < N_pruned <= N and 0 < K_pruned <= K):
        raise ValueError("N_pruned and K_pruned must lie in (0, N] and (0, K]")
    block_num = (N_pruned + N_DIM - 1) // N_DIM
    if block_num > MAX_BLOCK_NUM:
        raise ValueError(f"block_num = {block_num} exceeds {MAX_BLOCK_NUM}")
    N_ori, N_cal = reference_partition(N, N_pruned, N_DIM)
    if any(c > o for c, o in zip(N_cal, N_ori)):
        raise ValueError("a tile would keep more columns than it owns")
    K_cal = [K_pruned] * block_num
    off_B = [K * int(sum(N_ori[:t])) for t in range(block_num)]
    off_C = [M * int(sum(N_ori[:t])) for t in range(block_num)]

    dev = torch.device("cuda", torch.cuda.current_device())
    rng = np.random.Generator(np.random.PCG64(seed))
    A = torch.from_numpy(rng.random((K, M), dtype=np.float32) - 0.5).to(dev, dtype)      # [K][M]
    W = torch.from_numpy(rng.random((K, N), dtype=np.float32) - 0.5).to(dev, dtype)      # row-major K x N
    mk_h = [mask_gen(rng, K, K_cal[t]) for t in range(block_num)]
    mn_h = [mask_gen(rng, N_ori[t], N_cal[t]) for t in range(block_num)]
    mask_k = [torch.from_numpy(m).to(dev) for m in mk_h]
    mask_n = [torch.from_numpy(np.pad(m, (0, N_DIM - len(m)))).to(dev) for m in mn_h]

    # weights: zero-filled dense copy (baseline) and the compacted stream layout, built on the GPU
    W_pruned = torch.zeros_like(W)
    B_stream = torch.zeros((N, K), dtype=dtype, device=dev)        # column-major K x N, ldb = K
    rows_l, cols_l = [], []
    for t in range(block_num):
        rows = torch.from_numpy(mk_h[t] + np.arange(K_cal[t], dtype=np.int32)).to(dev, torch.long)
        cols = torch.from_numpy(mn_h[t] + np.arange(N_cal[t], dtype=np.int32) + off_C[t] // M).to(dev, torch.long)
        sub = W[rows][:, cols]
        W_pruned[rows[:, None], cols[None, :]] = sub
        base = off_C[t] // M
        B_stream[base:base + N_cal[t], :K_cal[t]] = sub.t()
        rows_l.append(rows)
        cols_l.append(cols)

    C_dense = torch.zeros((N, M), dtype=dtype, device=dev)
    C_stream = torch.zeros((N, M), dtype=dtype, device=dev)
    Wt = W_pruned.t().contiguous()

    def dense():
        torch.matmul(Wt, A, out=C_dense)

    stream = prepare_stream_gemm_nn(M, N, K, 1.0, A, B_stream, 0.0, C_stream, block_num, N_cal, K_cal, mask_n,
                                    mask_k, off_B, off_C)

    t_dense_warm = _time_us(dense, iters)
    print(f"CUTLASS GEMM : {t_dense_warm:f} us.", file=out)
    t_dense = _time_us(dense, iters)
    print(f"CUTLASS GEMM : {t_dense:f} us.", file=out)
    t_stream = _time_us(stream, iters)
    print(f"Stream  GEMM : {t_stream:f} us.", file=out)
    result = {"M": M, "N": N, "K": K, "N_pruned": N_pruned, "K_pruned": K_pruned, "block_num": block_num,
              "dense_us": t_dense, "stream_us": t_stream, "speedup": t_dense / t_stream,
              "kept_tflops": 2.0 * M * sum(n * k for n, k in zip(N_cal, K_cal)) / t_stream / 1e6, "errors": [],
              "errors_reference_rule": []}
    if check_results:
        # (ii) compaction + cuBLAS per tile (CuBlas_Gemm_NN_reference, basic_nn.cu:507-557)
        C_ref = torch.zeros((N, M), dtype=dtype, device=dev)
        for t in range(block_num):
            C_ref[cols_l[t]] = torch.matmul(W[rows_l[t]][:, cols_l[t]].t().contiguous(), A[rows_l[t]])
        result["errors"].append(checkout(C_stream, C_ref, err))
        result["errors_reference_rule"].append(checkout_counts(C_stream, C_ref, err)[1])
        # the CUDA-core twin through a layer handle built from the same index lists
        from .layer import TWLayer
        from .tiles import TileSet
        kp = np.concatenate([[0], np.cumsum(K_cal)]).astype(np.int32)
        npp = np.concatenate([[0], np.cumsum(N_cal)]).astype(np.int32)
        bounds = np.concatenate([[0], np.cumsum(N_ori)]).astype(np.int32)
        ts = TileSet(K, N, N_DIM, bounds, kp, torch.cat(rows_l).cpu().numpy().astype(np.int32), npp,
                     torch.cat(cols_l).cpu().numpy().astype(np.int32))
        layer = TWLayer(ts, dtype, dev)
        layer.pack(W)
        C_simt = layer.masked_gemm(A, simt=True)
        result["errors"].append(checkout(C_stream, C_simt, err))
        result["errors_reference_rule"].append(checkout_counts(C_stream, C_simt, err)[1])
        layer.close()
        # (iii) dense product on zero-filled weights
        result["errors"].append(checkout(C_stream, C_dense, err))
        result["errors_reference_rule"].append(checkout_counts(C_stream, C_dense, err)[1])
        print(f"elements only the magnitude guard lets through (reference rule to the letter): "
              f"{result['errors_reference_rule']} of {C_stream.numel()}", file=sys.stderr)
    return result


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="test_basic_nn", description=__doc__.split("\n")[0])
    ap.add_argument("M", type=int, nargs="?", default=768)
    ap.add_argument("N", type=int, nargs="?", default=768)
    ap.add_argument("K", type=int, nargs="?", default=768)
    ap.add_argument("N_pruned", type=int, nargs="?", default=None)
    ap.add_argument("K_pruned", type=int, nargs="?", default=None)
    ap.add_argument("--sparsity", type=float, default=None,
                    help="tile-wise sparsity in percent on K only: K_pruned = K*(1-s), N_pruned = N")
    ap.add_argument("--G", type=int, default=128, help="tile width; only 128 is supported, as in the reference")
    ap.add_argument("--dtype", choices=["f16", "bf16"], default="f16")
    ap.add_argument("--iters", type=int, default=100)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--no-check", action="store_true")
    a = ap.parse_args(argv)
    if a.G != 128:
        print("only G = 128 is supported by the driver", file=sys.stderr)
        return -1
    n_p = a.N_pruned if a.N_pruned is not None else (a.N if a.sparsity is not None else 768)
    k_p = a.K_pruned if a.K_pruned is not None else (
        int(round(a.K * (1 - a.sparsity / 100.0))) if a.sparsity is not None else 768)
    try:
        r = run(a.M, a.N, a.K, n_p, k_p, torch.bfloat16 if a.dtype == "bf16" else torch.float16, a.iters, a.seed,
                not a.no_check)
    except Exception as e:  # the reference driver reports failures through its exit code
        print(f"test_basic_nn failed: {e}", file=sys.stderr)
        return -1
    return 0 if not any(r["errors"]) else -1


if __name__ == "__main__":
    sys.exit(main())
