"""This library's masked GEMM against the REFERENCE's own kernel on the same seeded problem.

oracle/_ref/ref_stream_gemm (built by oracle/Makefile from oracle/ref_stream_gemm.cu and the
reference's unmodified CUTLASS headers) runs the reference's Volta884 masked GEMM the way its driver
does (StreamMaskedGEMM/perf/basic_nn.cu:411-427), on a problem read from a file.  The same problem goes
through ts_stream_gemm_nn.  The reference accumulates in fp16 (basic_nn.cu:250-259), this library in
fp32, so the two are compared with the driver's own tolerance err = 1e-2 (basic_nn.cu:1076-1077) and
both are held against the float64 product.  beta stays 0 as in the reference's driver: with beta != 0
the reference's tensor-core epilogue reads the source C without the column offsets it applies to the
store (cutlass/gemm/mma_epilogue.h:248-250), so its result there is not the masked product.
"""
import os
import struct
import subprocess

import numpy as np
import pytest
import torch

from oracle import masked_gemm as og

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_BIN = os.path.join(ROOT, "oracle", "_ref", "ref_stream_gemm")


def make_problem(M, N, K, N_pruned, K_pruned, seed, positive=False):
    from tilesparsity_b200.stream_gemm import mask_gen
    from tilesparsity_b200.tiles import reference_partition
    rng = np.random.Generator(np.random.PCG64(seed))
    bn = (N_pruned + 127) // 128
    N_ori, N_cal = reference_partition(N, N_pruned, 128)
    K_cal = [K_pruned] * bn
    off_B = [K * int(sum(N_ori[:t])) for t in range(bn)]
    off_C = [M * int(sum(N_ori[:t])) for t in range(bn)]
    shift = 0.0 if positive else 0.5
    A = (rng.random((K, M), dtype=np.float32) - shift).astype(np.float16)          # A^T, [K][M]
    W = ((rng.random((K, N), dtype=np.float32) - shift) * (0.05 if positive else 1.0)).astype(np.float16)
    mk = [mask_gen(rng, K, K_cal[t]) for t in range(bn)]
    mn = [mask_gen(rng, N_ori[t], N_cal[t]) for t in range(bn)]
    B = np.zeros((N, K), dtype=np.float16)                                         # column-major K x N, ldb = K
    rows_l, cols_l = [], []
    for t in range(bn):
        rows = mk[t] + np.arange(K_cal[t])
        cols = mn[t] + np.arange(N_cal[t]) + off_C[t] // M
        base = off_C[t] // M
        B[base:base + N_cal[t], :K_cal[t]] = W[np.ix_(rows, cols)].T
        rows_l.append(rows)
        cols_l.append(cols)
    return dict(M=M, N=N, K=K, bn=bn, N_cal=N_cal, K_cal=K_cal, off_B=off_B, off_C=off_C, A=A, W=W, B=B, mk=mk,
                mn=[np.pad(m, (0, 128 - len(m))).astype(np.int32) for m in mn], rows=rows_l, cols=cols_l)


def write_problem(path, p, alpha, beta, C0, iters):
    with open(path, "wb") as f:
        f.write(struct.pack("<6i", 0x54535247, p["M"], p["N"], p["K"], p["bn"], iters))
        for key in ("N_cal", "K_cal", "off_B", "off_C"):
            f.write(np.asarray(p[key], dtype=np.int32).tobytes())
        for t in range(p["bn"]):
            f.write(np.asarray(p["mk"][t], dtype=np.int32).tobytes())
            f.write(np.asarray(p["mn"][t], dtype=np.int32).tobytes())
        f.write(p["A"].tobytes())
        f.write(p["B"].tobytes())
        f.write(struct.pack("<2f", alpha, beta))
        f.write(C0.astype(np.float16).tobytes())


def run_reference_kernel(tmp_path, p, alpha, beta, C0, iters=0):
    prob, res = str(tmp_path / "problem.bin"), str(tmp_path / "result.bin")
    write_problem(prob, p, alpha, beta, C0, iters)
    r = subprocess.run([REF_BIN, prob, res], capture_output=True, text=True, timeout=180)
    assert r.returncode == 0, f"reference harness failed: {r.stdout}\n{r.stderr}"
    raw = np.fromfile(res, dtype=np.uint8)
    C = raw[:p["N"] * p["M"] * 2].view(np.float16).reshape(p["N"], p["M"])
    us = float(raw[p["N"] * p["M"] * 2:].view(np.float32)[0])
    return C, us


def run_this_library(p, alpha, beta, C0):
    from tilesparsity_b200.stream_gemm import stream_gemm_nn
    dev = torch.device("cuda", torch.cuda.current_device())
    A = torch.from_numpy(p["A"]).to(dev)
    B = torch.from_numpy(p["B"]).to(dev)
    C = torch.from_numpy(C0.astype(np.float16)).to(dev)
    mask_k = [torch.from_numpy(np.asarray(m, dtype=np.int32)).to(dev) for m in p["mk"]]
    mask_n = [torch.from_numpy(m).to(dev) for m in p["mn"]]
    stream_gemm_nn(p["M"], p["N"], p["K"], alpha, A, B, beta, C, p["bn"], p["N_cal"], p["K_cal"], mask_n, mask_k,
                   p["off_B"], p["off_C"])
    torch.cuda.synchronize()
    return C.cpu().numpy()


def exact_product(p, alpha, beta, C0):
    out = C0.astype(np.float64).copy()
    A64, W64 = p["A"].astype(np.float64), p["W"].astype(np.float64)
    for t in range(p["bn"]):
        r, c = p["rows"][t], p["cols"][t]
        out[c] = alpha * (W64[np.ix_(r, c)].T @ A64[r]) + beta * out[c]
    return out


needs_ref = pytest.mark.skipif(not os.path.exists(REF_BIN), reason="oracle/_ref/ref_stream_gemm is not built")


@needs_ref
@pytest.mark.parametrize("shape,alpha,beta", [((512, 768, 768, 384, 384), 1.0, 0.0),
                                              ((1000, 768, 3072, 384, 1536), 1.0, 0.0),
                                              ((256, 1024, 512, 1000, 136), 0.5, 0.0)])
def test_same_result_as_the_reference_kernel(tmp_path, shape, alpha, beta):
    M, N, K, Np, Kp = [(v + 7) // 8 * 8 for v in shape]
    p = make_problem(M, N, K, Np, Kp, seed=sum(shape))
    g = np.random.Generator(np.random.PCG64(1))
    C0 = (g.standard_normal((N, M)) if beta != 0 else np.zeros((N, M))).astype(np.float16)
    ref_c, _ = run_reference_kernel(tmp_path, p, alpha, beta, C0)
    mine = run_this_library(p, alpha, beta, C0)
    exact = exact_product(p, alpha, beta, C0)
    kept = np.concatenate(p["cols"])
    # both kernels against the float64 product: this library (fp32 accumulation) must be at least as
    # close as the reference (fp16 accumulation), and within the acceptance bound
    err_ref = og.max_rel_error(ref_c[kept], exact[kept])
    err_mine = og.max_rel_error(mine[kept], exact[kept])
    assert err_mine <= 1e-2 and err_mine <= err_ref + 1e-4, (err_mine, err_ref)
    # the two kernels against each other, the driver's tolerance on the matrix scale
    assert og.max_rel_error(mine[kept], ref_c[kept].astype(np.float64)) <= 1e-2
    # columns no tile keeps are left alone by both
    dead = np.setdiff1d(np.arange(N), kept)
    assert np.array_equal(mine[dead], C0[dead]) and np.array_equal(ref_c[dead], C0[dead])


@needs_ref
def test_reference_drivers_rule_between_the_two_kernels_on_positive_data(tmp_path):
    """checkout (basic_nn.cu:771-798) to the letter, reference kernel vs this library, on operands
    that do not cancel (where its ratio and absolute tests both mean something)."""
    p = make_problem(512, 768, 768, 384, 192, seed=77, positive=True)
    C0 = np.zeros((768, 512), dtype=np.float16)
    ref_c, _ = run_reference_kernel(tmp_path, p, 1.0, 0.0, C0)
    mine = run_this_library(p, 1.0, 0.0, C0)
    kept = np.concatenate(p["cols"])
    assert og.checkout_errors(mine[kept], ref_c[kept], 1e-2) == 0


@needs_ref
@pytest.mark.parametrize("shape", [(12800, 768, 768, 384, 384), (12800, 3072, 768, 1536, 384), (12800, 768, 3072, 384, 1536)])
def test_readme_shapes_agree_and_report_both_kernels_times(tmp_path, shape, capsys):
    """The shapes the reference's README quotes (StreamMaskedGEMM/README.md:14-27): results agree, and
    the microseconds of both kernels on this GPU are printed (run with -s to see them): the reference's
    kernel timed its own way (a stream per tile, a device synchronisation per pass, mean of 20 passes),
    this library's entry point with CUDA events over 20 back-to-back calls."""
    M, N, K, Np, Kp = shape
    p = make_problem(M, N, K, Np, Kp, seed=sum(shape))
    C0 = np.zeros((N, M), dtype=np.float16)
    ref_c, ref_us = run_reference_kernel(tmp_path, p, 1.0, 0.0, C0, iters=20)
    mine = run_this_library(p, 1.0, 0.0, C0)
    kept = np.concatenate(p["cols"])
    assert og.max_rel_error(mine[kept], ref_c[kept].astype(np.float64)) <= 1e-2
    from tilesparsity_b200.stream_gemm import prepare_stream_gemm_nn
    dev = torch.device("cuda", torch.cuda.current_device())
    A, B = torch.from_numpy(p["A"]).to(dev), torch.from_numpy(p["B"]).to(dev)
    C = torch.zeros((N, M), dtype=torch.float16, device=dev)
    mk = [torch.from_numpy(np.asarray(m, dtype=np.int32)).to(dev) for m in p["mk"]]
    mn = [torch.from_numpy(m).to(dev) for m in p["mn"]]
    call = prepare_stream_gemm_nn(M, N, K, 1.0, A, B, 0.0, C, p["bn"], p["N_cal"], p["K_cal"], mn, mk, p["off_B"], p["off_C"])
    for _ in range(3):
        call()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(20):
        call()
    e1.record()
    torch.cuda.synchronize()
    mine_us = e0.elapsed_time(e1) * 1e3 / 20
    with capsys.disabled():
        print(f"\nREADME shape M={M} N={N} K={K} N_pruned={Np} K_pruned={Kp}: reference kernel {ref_us:.1f} us, "
              f"this library {mine_us:.1f} us ({ref_us / mine_us:.1f}x)")
    assert ref_us > 0 and mine_us > 0
