"""Tensor-core masked GEMM (through the C ABI) vs the CPU oracle and vs its CUDA-core twin.

Acceptance, against the float32/float64 oracle evaluated on the same 16-bit-rounded inputs (fp16/bf16
inputs, fp32 accumulation): the matrix-level bound max |C - C_ref| / max |C_ref| <= 1e-2 AND the
per-element bound |C - C_ref| <= 1e-2 |C_ref| + 1e-3 rms(C_ref) on every element; the reference
driver's own rule (basic_nn.cu:785) is applied where its absolute test is meaningful (positive data).
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


def _accept(out, ref):
    assert og.max_rel_error(out, ref) <= TOL
    bad = og.elementwise_violations(out, ref, rtol=1e-2, floor=1e-3)
    assert bad == 0, f"{bad} of {ref.size} elements outside |err| <= 1e-2 |ref| + 1e-3 rms(ref)"


@pytest.mark.parametrize("K,N,M,keep,dtype,col_keep", CASES)
@pytest.mark.parametrize("unit_rows", [128, 256, 0])
def test_matches_oracle(K, N, M, keep, dtype, col_keep, unit_rows):
    layer, At, A16, W16 = _case(K, N, M, keep, dtype, K + N + M, col_keep)
    layer.set_unit_rows(unit_rows)              # both kernel variants, and the scheduler's own choice
    ref = og.masked_matmul_compacted(A16, W16, layer.tiles)
    Ct = layer.masked_gemm(At)
    layer.check()
    out = Ct.float().cpu().numpy()
    _accept(out, ref)
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
    """A batch with a ragged tail (M = 2048 + 72), beta != 0 through the host path, zeros in the
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


def test_host_buffer_calls_queued_back_to_back_on_one_layer():
    """Several asynchronous host-buffer calls on the same layer without a wait in between (different
    inputs, outputs alternating between two host buffers, a change of batch size in the middle): the
    library's events hand the staging buffers from call to call, one wait at the end suffices."""
    layer, At, A16, W16 = _case(512, 640, 1024, lambda g, nt: [128 + 32 * (t % 3) for t in range(nt)], torch.float16, 41)
    g = synth.rng(41)
    hAs, hCs, refs = [], [], []
    for i, M in enumerate((1024, 1024, 512, 1024, 1024)):
        a = torch.from_numpy(g.standard_normal((512, M), dtype=np.float32)).to(torch.float16)
        hAs.append(a.pin_memory())
        hCs.append(torch.full((640, M), 7.0, dtype=torch.float16).pin_memory())
        refs.append(og.masked_matmul_compacted(a.float().numpy(), W16, layer.tiles))
    for a, c in zip(hAs, hCs):
        layer.masked_gemm_host(a, c, wait=False)
    layer.host_wait()
    torch.cuda.current_stream().synchronize()
    for c, ref in zip(hCs, refs):
        _accept(c.float().numpy(), ref)
    layer.check()
    layer.close()


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_split_k_units_match_the_oracle_and_the_unsplit_schedule(dtype):
    """A layer with one long tile beside light ones (the VGG conv5 "10 % columns + 75 % rows" pattern):
    the long tile's kept rows run as several units per batch block whose fp32 partial sums a second
    kernel adds up.  Checked against the oracle, with bias + activation and with beta, with a ragged
    batch, and against the same layer with split-K turned off."""
    from tilesparsity_b200 import TWLayer
    from tilesparsity_b200.tiles import tiles_from_lists
    g = synth.rng(91)
    K, N, M = 4608, 512, 2048 + 64
    col = np.ones(N, bool)
    col[g.choice(N, size=52, replace=False)] = False            # 460 kept columns: 3 full tiles + 76
    nt = len(tile_bounds_from_col_mask(col, 128)) - 1
    counts = [87, 155, 91, 4275][:nt]
    lists = [np.sort(g.permutation(K)[:c]).astype(np.int32) for c in counts]
    parts = np.zeros(nt, np.int32)
    import ctypes as C
    from tilesparsity_b200 import _lib
    p32 = lambda a: a.ctypes.data_as(C.POINTER(C.c_int32))
    b = tile_bounds_from_col_mask(col, 128)
    ncols = np.array([col[b[t]:b[t + 1]].sum() for t in range(nt)], np.int32)
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    _lib.check(_lib.lib.ts_plan_split(nt, p32(np.asarray(counts, np.int32)), p32(ncols), K, M, sms, p32(parts)))
    assert parts.max() > 1, "the case is meant to exercise split units"
    W = (g.standard_normal((K, N), dtype=np.float32) * np.float32(0.02)).astype(np.float32)
    Wd = torch.from_numpy(W).cuda()
    A = g.standard_normal((K, M), dtype=np.float32)
    At = torch.from_numpy(A).to(dtype).cuda()
    A16, W16 = At.float().cpu().numpy(), Wd.to(dtype).float().cpu().numpy()
    layer = TWLayer.from_lists(Wd, lists, col, 128, dtype)
    ref = og.masked_matmul_compacted(A16, W16, layer.tiles)
    C1 = layer.masked_gemm(At)
    _accept(C1.float().cpu().numpy(), ref)
    assert not C1.float().cpu().numpy()[~col].any()
    # epilogue: bias + relu, then alpha / beta on top of an existing output
    bias = torch.from_numpy(g.standard_normal(N, dtype=np.float32)).cuda()
    C2 = layer.masked_gemm(At, bias=bias, activation="relu")
    ref2 = np.maximum(ref + bias.cpu().numpy()[:, None], 0.0) * col[:, None]
    _accept(C2.float().cpu().numpy(), ref2)
    C3 = C1.clone()
    layer.masked_gemm(At, out=C3, alpha=0.5, beta=1.0)
    _accept(C3.float().cpu().numpy(), 1.5 * ref)
    # deterministic, and equal to the unsplit schedule within the rounding of one 16-bit result
    assert torch.equal(layer.masked_gemm(At), C1)
    layer.set_split_k(False)
    C4 = layer.masked_gemm(At)
    _accept(C4.float().cpu().numpy(), ref)
    assert og.max_rel_error(C4.float().cpu().numpy(), C1.float().cpu().numpy()) <= (4e-3 if dtype == torch.bfloat16 else 1e-3)
    layer.check()
    layer.close()


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


# ------------------------------------------------------------------------------------------------
# The benchmark configurations at their own sizes
# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("name", ["qkv", "attn_out", "ffn1", "ffn2"])
@pytest.mark.parametrize("sparsity", [50.0, 75.0, 90.0])
def test_bert_layer_gemms_with_gpu_built_tw1_masks(name, sparsity):
    """BERT-base GEMMs at M = 4096, fp16, with the tw1 masks the GPU mask builder derives from the
    synthetic weights (non-uniform kept rows per tile): the workload bench.py times."""
    from tilesparsity_b200 import TWLayer, build_mask
    A, W = synth.bert_gemm(name, 4096)
    Wd = torch.from_numpy(W).cuda()
    res = build_mask("tw1", [Wd.abs()], sparsity, 128)
    layer = TWLayer(res.tiles[0], torch.float16, Wd.device)
    layer.pack(Wd)
    At = torch.from_numpy(np.ascontiguousarray(A.T)).to(torch.float16).cuda()
    out = layer.masked_gemm(At).float().cpu().numpy()
    layer.check()
    ref = og.masked_matmul_compacted(At.float().cpu().numpy(), Wd.half().float().cpu().numpy(), layer.tiles)
    _accept(out, ref)
    # the dense-masked form the reference's model code computes (modeling.py:1001-1003)
    mask = res.masks[0].cpu().numpy()
    dense = og.masked_matmul_dense(At.float().cpu().numpy().T, Wd.half().float().cpu().numpy(), mask).T
    _accept(out, dense)
    layer.close()


@pytest.mark.parametrize("algo,sparsity,g1", [("tw2", 75.0, None), ("tw_cols_rows", 75.0, 10.0)])
def test_vgg_conv5_shape_at_full_batch(algo, sparsity, g1):
    """VGG16 conv5 as a GEMM: M = 64 x 14 x 14 = 12544, K = 4608, N = 512, bf16, activations after a
    ReLU (about half zeros), He-normal weights; the reference's tw2 at 75 % and the "10 % of the
    columns, then 75 % of the rows" mask, both built by the GPU mask builder."""
    from tilesparsity_b200 import TWLayer, build_mask
    g = synth.rng(3001)
    M, K, N = 12544, 4608, 512
    A = np.maximum(g.standard_normal((M, K), dtype=np.float32), 0)
    W = g.standard_normal((K, N), dtype=np.float32) * np.float32(np.sqrt(2.0 / K))
    Wd = torch.from_numpy(W).cuda()
    res = build_mask(algo, [Wd.abs()], sparsity, 128, g1)
    ts = res.tiles[0]
    if algo == "tw_cols_rows":
        want = om_tw_cols_rows(np.abs(W), g1, sparsity)
        assert np.array_equal(res.masks[0].cpu().numpy(), want)
        assert abs(ts.col_mask().mean() - 0.9) < 0.01
    layer = TWLayer(ts, torch.bfloat16, Wd.device)
    layer.pack(Wd)
    At = torch.from_numpy(np.ascontiguousarray(A.T)).to(torch.bfloat16).cuda()
    out = layer.masked_gemm(At).float().cpu().numpy()
    layer.check()
    ref = og.masked_matmul_compacted(At.float().cpu().numpy(), Wd.bfloat16().float().cpu().numpy(), ts)
    _accept(out, ref)
    assert not out[~ts.col_mask()].any()
    layer.close()


def om_tw_cols_rows(score, col_sparsity, row_sparsity):
    from oracle import tw_masks as om
    return np.asarray(om.tw_cols_rows([score], col_sparsity, row_sparsity, 128)[0], dtype=bool)


def test_nmt_lstm_tew_at_config_size():
    """NMT LSTM gate GEMM: K = 2048, N = 4096, M = 6400, fp16, W ~ U(-0.1, 0.1), TEW = tw1m at 75 % with
    a 1.5 % element-wise residual kept as a sparse term; against A @ (W * mask_tew)."""
    from tilesparsity_b200 import TEWLayer, build_mask
    g = synth.rng(4001)
    K, N, M = 2048, 4096, 6400
    W = g.uniform(-0.1, 0.1, size=(K, N)).astype(np.float32)
    A = g.standard_normal((M, K), dtype=np.float32)
    Wd = torch.from_numpy(W).cuda()
    res = build_mask("tw1m", [Wd.abs()], 75.0, 128, 1.5, want_residual=True)
    layer = TEWLayer(Wd, res.tiles[0], res.residuals[0], torch.float16)
    assert abs(layer.nnz / (K * N) - 0.015) < 0.002
    At = torch.from_numpy(np.ascontiguousarray(A.T)).to(torch.float16).cuda()
    out = layer.masked_gemm(At).float().cpu().numpy()
    layer.tw.check()
    mask = res.masks[0].cpu().numpy()
    ref = og.masked_matmul_dense(At.float().cpu().numpy().T, Wd.half().float().cpu().numpy(), mask).T
    _accept(out, ref)
    layer.close()


@pytest.mark.parametrize("n", [4096, 8192])
def test_skewed_squares_against_the_oracle_on_sampled_rows(n):
    """M = N = K = n, bf16, per-tile kept-row counts ~ Beta(2,5): 96 output rows (two per sampled tile
    plus random ones) against the float64 oracle; the whole output against the CUDA-core twin."""
    from tilesparsity_b200 import TWLayer
    from tilesparsity_b200.tiles import tiles_from_lists
    nt = n // 128
    counts = synth.beta_skewed_counts(n, nt, 0.25, 5000 + int(np.log2(n)))
    g = synth.rng(5000 + int(np.log2(n)))
    lists = [np.sort(g.choice(n, size=int(c), replace=False)).astype(np.int32) for c in counts]
    ts = tiles_from_lists(n, n, 128, lists)
    gen = torch.Generator(device="cuda").manual_seed(n)
    W = torch.randn((n, n), generator=gen, device="cuda", dtype=torch.float32)
    At = torch.randn((n, n), generator=gen, device="cuda", dtype=torch.float32).to(torch.bfloat16)
    layer = TWLayer(ts, torch.bfloat16, W.device)
    layer.pack(W)
    out = layer.masked_gemm(At)
    layer.check()
    heavy, light = int(np.argmax(counts)), int(np.argmin(counts))
    rows = sorted(set([heavy * 128, heavy * 128 + 127, light * 128, light * 128 + 5] +
                      [int(r) for r in g.choice(n, size=92, replace=False)]))
    ref = og.masked_matmul_rows(At.float().cpu().numpy(), W.bfloat16().float().cpu().numpy(), ts, rows)
    got = out[torch.tensor(rows, device="cuda")].float().cpu().numpy()
    _accept(got, ref)
    if n <= 4096:
        twin = layer.masked_gemm(At, simt=True).float()
        assert float((out.float() - twin).abs().max() / twin.abs().max()) <= TOL
    layer.close()


def test_reference_drivers_acceptance_rule_on_positive_data():
    """The perf driver's `checkout` (basic_nn.cu:771-798: ratio either way > 1 + err, or |diff| > err,
    err = 1e-2) with no relaxation, on operands that do not cancel."""
    from tilesparsity_b200 import TWLayer
    g = synth.rng(123)
    K, N, M = 768, 1024, 1024
    A = g.random((M, K), dtype=np.float32)
    W = g.random((K, N), dtype=np.float32) * np.float32(0.05)
    lists = synth.random_kept_lists(K, N // 128, 192, 124)
    Wd = torch.from_numpy(W).cuda()
    layer = TWLayer.from_lists(Wd, lists, None, 128, torch.float16)
    At = torch.from_numpy(np.ascontiguousarray(A.T)).to(torch.float16).cuda()
    out = layer.masked_gemm(At).float().cpu().numpy()
    ref = og.masked_matmul_compacted(At.float().cpu().numpy(), Wd.half().float().cpu().numpy(), layer.tiles)
    assert og.checkout_errors(out, ref, 1e-2) == 0
    layer.close()


def test_host_buffer_path_returns_zeros_in_pruned_columns_after_m_or_tiles_change():
    """The staging output of the host-buffer entry point is zeroed lazily: a different batch size (the
    row pitch changes) or a different tile set must not let earlier results show through in the
    columns no tile keeps."""
    from tilesparsity_b200 import TWLayer
    from tilesparsity_b200.tiles import tiles_from_lists
    g = synth.rng(77)
    K, N = 256, 512
    W = (g.standard_normal((K, N), dtype=np.float32) * np.float32(0.05)).astype(np.float32)
    Wd = torch.from_numpy(W).cuda()
    col1 = g.random(N) < 0.7
    col2 = g.random(N) < 0.5

    def lists_for(col):
        nt = len(tile_bounds_from_col_mask(col, 128)) - 1
        return synth.random_kept_lists(K, nt, 64, int(col.sum()))

    layer = TWLayer.from_lists(Wd, lists_for(col1), col1, 128, torch.float16)
    for M in (512, 256, 384):
        hA = torch.from_numpy(g.standard_normal((K, M), dtype=np.float32)).to(torch.float16).pin_memory()
        hC = torch.full((N, M), 9.0, dtype=torch.float16).pin_memory()
        layer.masked_gemm_host(hA, hC)
        ref = og.masked_matmul_compacted(hA.float().numpy(), Wd.half().float().cpu().numpy(), layer.tiles)
        _accept(hC.float().numpy(), ref)
        assert not hC.numpy()[~col1].any(), f"stale values in pruned columns at M = {M}"
    layer.close()
    # the same handle re-used with another tile set
    layer = TWLayer.from_lists(Wd, lists_for(col1), col1, 128, torch.float16)
    hA = torch.from_numpy(g.standard_normal((K, 256), dtype=np.float32)).to(torch.float16).pin_memory()
    hC = torch.empty((N, 256), dtype=torch.float16).pin_memory()
    layer.masked_gemm_host(hA, hC)
    ts2 = tiles_from_lists(K, N, 128, lists_for(col2), col2)
    layer.retile(ts2)
    layer.pack(Wd)
    layer.masked_gemm_host(hA, hC)
    ref = og.masked_matmul_compacted(hA.float().numpy(), Wd.half().float().cpu().numpy(), ts2)
    _accept(hC.float().numpy(), ref)
    assert not hC.numpy()[~col2].any()
    layer.close()
