"""Tensor-core masked GEMM (through the C ABI) vs the CPU oracle and vs its CUDA-core twin.

Acceptance bound: max |C - C_ref| / max |C_ref| <= 1e-2 against the float32 oracle evaluated on the
same 16-bit-rounded inputs (fp16/bf16 inputs, fp32 accumulation).
"""
import numpy as np
import pytest
import torch

from oracle import masked_gemm as og
from tilesparsity_b200 import synth
from tilesparsity_b200.tiles import tile_bounds_from_col_mask

pytestmark = pytest.mark.gpu
TOL = 1e-2


def _case(K, N, M, keep, dtype, seed, col_keep=None, scale=0.05):
    from tilesparsity_b200 import TWLayer
    g = synth.rng(seed)
    A = g.standard_normal((M, K), dtype=np.float32)
    W = (g.standard_normal((K, N), dtype=np.float32) * np.float32(scale)).astype(np.float32)
    col = (g.random(N) < col_keep) if col_keep is not None else None
    nt = len(tile_bounds_from_col_mask(np.ones(N, bool) if col is None else col, 128)) - 1
    if callable(keep):
        counts = keep(g, nt)
    else:
        counts = [keep] * nt
    lists = [np.sort(g.permutation(K)[:int(c)]).astype(np.int32) for c in counts]
    Wd = torch.from_numpy(W).cuda()
    layer = TWLayer.from_lists(Wd, lists, col, 128, dtype)
    At = torch.from_numpy(np.ascontiguousarray(A.T)).to(dtype).cuda()
    A16 = At.float().cpu().numpy()
    W16 = Wd.to(dtype).float().cpu().numpy()
    return layer, At, A16, W16


CASES = [
    # K, N, M, kept rows per tile, dtype, column keep fraction
    (64, 128, 8, 64, torch.float16, None),            # a single tile, everything kept, tiny batch
    (64, 128, 256, 16, torch.float16, None),
    (256, 128, 264, 192, torch.float16, None),        # batch tail (264 = 256 + 8)
    (256, 256, 512, 100, torch.bfloat16, None),       # kept rows not a multiple of 16
    (768, 768, 1000, 192, torch.float16, None),       # M not a multiple of the unit
    (768, 3072, 4096, 192, torch.float16, None),      # BERT FFN1 at 75 %
    (3072, 768, 4096, 768, torch.bfloat16, None),     # BERT FFN2 at 75 %
    (768, 2304, 4096, 384, torch.float16, None),      # BERT QKV at 50 %
    (768, 768, 4096, 80, torch.float16, None),        # BERT attention output at ~90 %
    (512, 700, 520, 33, torch.float16, 0.6),          # pruned columns: scattered output rows, ragged last tile
    (4608, 512, 1024, 1152, torch.bfloat16, 0.9),     # VGG conv5 as GEMM, 75 % rows + 10 % columns
]


@pytest.mark.parametrize("K,N,M,keep,dtype,col_keep", CASES)
@pytest.mark.parametrize("unit_rows", ["128", "256"])
def test_matches_oracle(K, N, M, keep, dtype, col_keep, unit_rows, monkeypatch):
    monkeypatch.setenv("TS_UNIT_ROWS", unit_rows)
    layer, At, A16, W16 = _case(K, N, M, keep, dtype, K + N + M, col_keep)
    ref = og.masked_matmul_compacted(A16, W16, layer.tiles)
    Ct = layer.masked_gemm(At)
    layer.check()
    out = Ct.float().cpu().numpy()
    assert og.max_rel_error(out, ref) <= TOL
    # columns no tile keeps are untouched (the output buffer starts as zeros)
    dead = ~layer.tiles.col_mask()
    assert not out[dead].any()
    # the packed weights are exactly the compaction of the 16-bit weights
    wp = layer.packed_weights().float().numpy()
    assert np.array_equal(wp, og.pack_weights(W16, layer.tiles, ld=wp.shape[1]))
    layer.close()


def test_ragged_kept_counts_and_empty_tiles():
    def counts(g, nt):
        c = g.integers(0, 300, nt)
        c[0] = 0                      # a tile without kept rows still writes zeros
        c[-1] = 1
        return c
    layer, At, A16, W16 = _case(768, 1536, 2048, counts, torch.bfloat16, 99)
    ref = og.masked_matmul_compacted(A16, W16, layer.tiles)
    out_t = torch.full((1536, 2048), 7.0, dtype=torch.bfloat16, device="cuda")
    layer.masked_gemm(At, out=out_t)
    layer.check()
    out = out_t.float().cpu().numpy()
    assert og.max_rel_error(out, ref) <= TOL
    assert not out[layer.tiles.tile_cols(0)].any()
    layer.close()


def test_alpha_beta():
    layer, At, A16, W16 = _case(256, 384, 512, 64, torch.float16, 5, col_keep=0.8)
    g = synth.rng(6)
    C0 = torch.from_numpy(g.standard_normal((384, 512), dtype=np.float32)).to(torch.float16).cuda()
    ref = og.masked_matmul_compacted(A16, W16, layer.tiles, alpha=0.5, beta=-1.5, Ct=C0.float().cpu().numpy())
    out = layer.masked_gemm(At, out=C0.clone(), alpha=0.5, beta=-1.5).float().cpu().numpy()
    assert og.max_rel_error(out, ref) <= TOL
    dead = ~layer.tiles.col_mask()
    assert np.array_equal(out[dead], C0.float().cpu().numpy()[dead])
    layer.close()


def test_tensor_core_and_cuda_core_paths_agree_on_a_large_shape():
    # too large for the CPU oracle to be quick: the CUDA-core twin is the checker
    layer, At, _, _ = _case(4096, 4096, 4096, lambda g, nt: synth.beta_skewed_counts(4096, nt, 0.25, 5012), torch.bfloat16, 12)
    a = layer.masked_gemm(At).float()
    b = layer.masked_gemm(At, simt=True).float()
    layer.check()
    assert float((a - b).abs().max() / b.abs().max()) <= TOL
    st = layer.schedule_stats(4096)
    assert st["n_units"] >= layer.tiles.n_tiles * 16 and 0.5 < st["balance"] <= 1.0
    layer.close()


def test_deterministic_and_linear():
    layer, At, A16, W16 = _case(768, 768, 1024, 192, torch.float16, 21)
    c1 = layer.masked_gemm(At)
    c2 = layer.masked_gemm(At)
    assert torch.equal(c1, c2)
    c3 = layer.masked_gemm(At * 2)
    assert float((c3.float() - 2 * c1.float()).abs().max()) <= 2e-3 * float(c1.float().abs().max())
    layer.close()


def test_host_buffer_entry_point_and_row_major_op():
    from tilesparsity_b200 import masked_linear
    layer, At, A16, W16 = _case(768, 768, 512, 192, torch.float16, 31)
    ref = og.masked_matmul_compacted(A16, W16, layer.tiles)
    hA = At.cpu().pin_memory()
    hC = torch.empty((768, 512), dtype=torch.float16).pin_memory()
    layer.masked_gemm_host(hA, hC)
    assert og.max_rel_error(hC.float().numpy(), ref) <= TOL
    C_rm = masked_linear(At.t().contiguous(), layer)
    assert og.max_rel_error(C_rm.float().cpu().numpy().T, ref) <= TOL
    layer.close()


def test_host_buffer_pipeline_blocks_beta_and_async():
    """Four column blocks (M = 2048 + a ragged tail), beta != 0 through the host path, zeros in the
    columns no tile keeps after a beta pass, and the asynchronous variant on two layers at once."""
    M = 2048 + 72
    layer, At, A16, W16 = _case(384, 512, M, 96, torch.float16, 33)
    ref = og.masked_matmul_compacted(A16, W16, layer.tiles)
    hA = At.cpu().pin_memory()
    hC = torch.empty((512, M), dtype=torch.float16).pin_memory()
    layer.masked_gemm_host(hA, hC)
    assert og.max_rel_error(hC.float().numpy(), ref) <= TOL
    first = hC.clone()
    layer.masked_gemm_host(hA, hC, alpha=0.5, beta=1.0)            # C <- 0.5 A W + C
    assert og.max_rel_error(hC.float().numpy(), 1.5 * ref) <= TOL
    layer.masked_gemm_host(hA, hC)                                   # beta = 0 again
    assert torch.equal(hC, first)
    layer2, At2, A2, W2 = _case(256, 384, M, 64, torch.float16, 34)
    ref2 = og.masked_matmul_compacted(A2, W2, layer2.tiles)
    hA2 = At2.cpu().pin_memory()
    hC2 = torch.empty((384, M), dtype=torch.float16).pin_memory()
    hC.zero_()
    layer.masked_gemm_host(hA, hC, wait=False)
    layer2.masked_gemm_host(hA2, hC2, wait=False)
    layer.host_wait()
    layer2.host_wait()
    torch.cuda.current_stream().synchronize()
    assert torch.equal(hC, first)
    assert og.max_rel_error(hC2.float().numpy(), ref2) <= TOL
    layer.close()
    layer2.close()


def test_grouped_layers_equal_separate_launches():
    """Independent layers as one block-structured layer over stacked activations and outputs."""
    from tilesparsity_b200 import TWLayer
    M = 512
    a, At_a, _, _ = _case(256, 384, M, 64, torch.float16, 51)
    b, At_b, _, _ = _case(640, 128, M, lambda g, nt: [200] * nt, torch.float16, 52)
    g1, g2 = synth.rng(51), synth.rng(52)
    # the dense weights the two cases were packed from
    g1.standard_normal((M, 256), dtype=np.float32)
    Wa = torch.from_numpy((g1.standard_normal((256, 384), dtype=np.float32) * np.float32(0.05))).cuda()
    g2.standard_normal((M, 640), dtype=np.float32)
    Wb = torch.from_numpy((g2.standard_normal((640, 128), dtype=np.float32) * np.float32(0.05))).cuda()
    layer, k_off, n_off = TWLayer.grouped([Wa, Wb], [a.tiles, b.tiles], torch.float16)
    out = layer.masked_gemm(torch.cat([At_a, At_b], dim=0).contiguous())
    assert torch.equal(out[:384], a.masked_gemm(At_a))
    assert torch.equal(out[384:], b.masked_gemm(At_b))
    for x in (layer, a, b):
        x.close()


def test_bad_arguments_are_rejected():
    from tilesparsity_b200 import TileSparseError
    layer, At, _, _ = _case(64, 128, 64, 16, torch.float16, 41)
    with pytest.raises(ValueError):
        layer.masked_gemm(At[:, :60].contiguous().to(torch.bfloat16))
    with pytest.raises(TileSparseError):
        layer.masked_gemm(At[:, :60].contiguous())          # M = 60 is not a multiple of 8
    layer.close()


def test_tile_sharded_layers_reproduce_the_unsharded_output():
    """World of 3 emulated on one GPU: each rank's share runs by itself, slabs are joined by hand."""
    from tilesparsity_b200 import TWLayer, sharding
    layer, At, A16, W16 = _case(512, 1700, 512, lambda g, nt: synth.beta_skewed_counts(512, nt, 0.25, 3),
                                torch.float16, 55, col_keep=0.85)
    full = layer.masked_gemm(At)
    Wd = torch.from_numpy(W16).cuda()
    world = 3
    slabs, shard = [], None
    for r in range(world):
        shard = sharding.ShardedTWLayer(Wd, layer.tiles, r, world, torch.float16)
        slabs.append(shard.masked_gemm(At))
        assert shard.plan.balance() > 0.8
    joined = shard.assemble(torch.cat(slabs, 0))
    assert torch.equal(joined, full)
    layer.close()


@pytest.mark.parametrize("algo,shape,sparsity,g1", [("tw1m", (512, 1024), 75.0, 1.5), ("tw2m", (384, 768), 60.0, 2.0)])
def test_tew_layer_matches_the_dense_masked_product(algo, shape, sparsity, g1):
    """TW part on the tensor cores + residual as a sparse term == A @ (W * mask_tew)."""
    from tilesparsity_b200 import TEWLayer, build_mask
    g = synth.rng(sum(shape))
    K, N = shape
    M = 520
    W = g.uniform(-0.1, 0.1, size=shape).astype(np.float32)
    A = g.standard_normal((M, K), dtype=np.float32)
    res = build_mask(algo, [np.abs(W)], sparsity, 128, g1, want_residual=True)
    Wd = torch.from_numpy(W).cuda()
    layer = TEWLayer(Wd, res.tiles[0], res.residuals[0], torch.float16)
    assert layer.nnz > 0
    At = torch.from_numpy(np.ascontiguousarray(A.T)).to(torch.float16).cuda()
    out = layer.masked_gemm(At).float().cpu().numpy()
    mask = res.masks[0].cpu().numpy()
    ref = og.masked_matmul_dense(At.float().cpu().numpy().T, Wd.half().float().cpu().numpy(), mask).T
    assert og.max_rel_error(out, ref) <= TOL
    layer.close()


@pytest.mark.parametrize("act", [None, "relu", "gelu"])
@pytest.mark.parametrize("col_keep", [None, 0.8])
def test_fused_bias_and_activation(act, col_keep):
    """y = act(x @ (W * mask) + bias): mask_dense's bias add (modeling.py:1003-1007) and the layer's
    activation folded into the GEMM epilogue, on both store paths (TMA tile store / list-driven)."""
    layer, At, A16, W16 = _case(384, 640, 520, 96, torch.float16, 77, col_keep=col_keep)
    g = synth.rng(78)
    bias = g.standard_normal(640).astype(np.float32)
    ref = og.masked_matmul_compacted(A16, W16, layer.tiles) + bias[:, None]
    if act == "relu":
        ref = np.maximum(ref, 0)
    elif act == "gelu":
        ref = ref * 0.5 * (1.0 + np.tanh(np.sqrt(2 / np.pi) * (ref + 0.044715 * ref ** 3)))
    kept = layer.tiles.col_mask()
    out = layer.masked_gemm(At, bias=torch.from_numpy(bias).cuda(), activation=act).float().cpu().numpy()
    assert og.max_rel_error(out[kept], ref[kept]) <= TOL
    assert not out[~kept].any()
    layer.close()


def test_peer_copies_receive_the_same_rows():
    """The epilogue's extra destinations (the all-gather of a sharded layer) on one GPU: two more
    buffers must end up identical to the primary output."""
    layer, At, A16, W16 = _case(256, 512, 520, 64, torch.bfloat16, 91, col_keep=0.7)
    extra = [torch.zeros((512, 520), dtype=torch.bfloat16, device="cuda") for _ in range(2)]
    out = layer.masked_gemm(At, peers=[e.data_ptr() for e in extra])
    assert torch.equal(extra[0], out) and torch.equal(extra[1], out)
    layer.close()
