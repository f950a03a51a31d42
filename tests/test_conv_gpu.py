"""Implicit-GEMM convolution (ConvTWLayer) against the CPU oracle: im2col + the masked product.

The oracle builds the im2col matrix the reference's row order implies (img2col_forward,
Pruning/VGG/prune_algo.py:16-24) and multiplies it with W .* mask; the library never builds it."""
import numpy as np
import pytest
import torch

from oracle import masked_gemm as og
from tilesparsity_b200 import synth

pytestmark = pytest.mark.gpu


def _run(B, H, W, cin, cout, kh, kw, algo, sparsity, g1, dtype, seed, relu_in=True):
    from tilesparsity_b200 import ConvTWLayer, build_mask, masks
    g = synth.rng(seed)
    x = g.standard_normal((B, H, W, cin), dtype=np.float32)
    if relu_in:
        x = np.maximum(x, 0)
    w = (g.standard_normal((kh, kw, cin, cout), dtype=np.float32) * np.float32(np.sqrt(2.0 / (kh * kw * cin)))).astype(np.float32)
    wd = torch.from_numpy(w).cuda()
    scores = masks.img2col_forward([wd])
    res = build_mask(algo, scores, sparsity, 128, g1)
    layer = ConvTWLayer(wd, res.tiles[0], dtype)
    xd = torch.from_numpy(x).to(dtype).cuda()
    y = layer.forward(xd)
    layer.layer.check()
    x16 = xd.float().cpu().numpy()
    w16 = wd.to(dtype).float().cpu().numpy().reshape(-1, cout)
    ref = og.masked_matmul_dense(og.im2col_nhwc(x16, kh, kw), w16, res.masks[0].cpu().numpy()).reshape(B, H, W, cout)
    out = y.float().cpu().numpy()
    assert og.max_rel_error(out, ref) <= 1e-2
    assert og.elementwise_violations(out, ref, rtol=1e-2, floor=1e-3) == 0
    dead = ~res.tiles[0].col_mask()
    assert not out[..., dead].any()
    return layer, xd, y


@pytest.mark.parametrize("B,H,W,cin,cout,kh,kw,algo,sparsity,g1,dtype", [
    (2, 5, 7, 16, 40, 3, 3, "tw1", 50.0, None, torch.float16),            # ragged everything, one narrow tile
    (3, 14, 14, 64, 256, 3, 3, "tw2", 75.0, None, torch.bfloat16),         # pruned output channels
    (1, 9, 20, 32, 136, 5, 3, "tw1", 60.0, None, torch.float16),           # non-square kernel, Wp > W + kw - 1
    (4, 8, 8, 128, 128, 1, 1, "tw1", 75.0, None, torch.bfloat16),          # 1 x 1: a plain GEMM over pixels
    (1, 224, 224, 8, 16, 3, 3, "tw1", 50.0, None, torch.float16),          # ImageNet-sized image, 226 x 232 padded
    (2, 30, 41, 8, 24, 7, 5, "tw1", 40.0, None, torch.bfloat16),           # wide kernel, Wp / 8 and Hp not powers of two
])
def test_small_convolutions_match_the_oracle(B, H, W, cin, cout, kh, kw, algo, sparsity, g1, dtype):
    layer, _, _ = _run(B, H, W, cin, cout, kh, kw, algo, sparsity, g1, dtype, seed=B + H + W + cin)
    layer.close()


@pytest.mark.parametrize("algo,sparsity,g1", [("tw2", 75.0, None), ("tw_cols_rows", 75.0, 10.0)])
def test_vgg16_conv5_at_full_batch(algo, sparsity, g1):
    """Batch 64, 14 x 14, 3 x 3, 512 -> 512 channels, bf16, activations after a ReLU."""
    layer, xd, y = _run(64, 14, 14, 512, 512, 3, 3, algo, sparsity, g1, torch.bfloat16, seed=3001)
    assert tuple(y.shape) == (64, 14, 14, 512)
    # algorithmic bytes count the NHWC input once (12.85 MB), not an im2col matrix (115.6 MB)
    assert layer.algorithmic_bytes(64, 14, 14) < 40e6
    layer.close()


def test_geometry_and_bad_arguments():
    from tilesparsity_b200 import ConvTWLayer, TileSparseError, conv
    geo = conv.geometry(64, 14, 14, 3, 3)
    assert geo == {"Hp": 16, "Wp": 16, "m_padded": 64 * 256, "plane_ld": 64 * 256 + 32}
    geo = conv.geometry(1, 224, 224, 3, 3)
    assert geo["Wp"] == 232 and geo["Hp"] == 226
    from tilesparsity_b200.tiles import tiles_from_lists
    ts = tiles_from_lists(72, 128, 128, [np.arange(0, 72, 2, dtype=np.int32)])
    w = torch.zeros((3, 3, 8, 128), device="cuda")
    layer = ConvTWLayer(w, ts, torch.float16)
    with pytest.raises(ValueError):
        layer.pack_input(torch.zeros((1, 4, 4, 9), dtype=torch.float16, device="cuda"))
    layer.close()
    with pytest.raises(ValueError):
        ConvTWLayer(torch.zeros((3, 3, 4, 128), device="cuda"), ts, torch.float16)
    with pytest.raises(TileSparseError):
        conv.geometry(0, 4, 4, 3, 3)


@pytest.mark.parametrize("kh,kw,B,H,W", [(3, 3, 2, 6, 10), (5, 5, 1, 9, 13), (3, 7, 2, 5, 17), (1, 9, 1, 4, 23), (1, 1, 3, 5, 6)])
def test_two_convolutions_chained_in_the_padded_layout(kh, kw, B, H, W):
    """conv -> ReLU -> conv without an NHWC round trip: the first layer's padded-space output goes
    through ts_conv_repack straight into the second layer's input planes (every kernel width the pack
    and repack kernels are instantiated for)."""
    from tilesparsity_b200 import ConvTWLayer, build_mask, masks
    g = synth.rng(909 + kh * 10 + kw)
    c0, c1, c2 = 32, 64, 128
    x = np.maximum(g.standard_normal((B, H, W, c0), dtype=np.float32), 0)
    w1 = (g.standard_normal((kh, kw, c0, c1), dtype=np.float32) * np.float32(np.sqrt(2.0 / (kh * kw * c0)))).astype(np.float32)
    w2 = (g.standard_normal((kh, kw, c1, c2), dtype=np.float32) * np.float32(np.sqrt(2.0 / (kh * kw * c1)))).astype(np.float32)
    dt = torch.float16
    wd1, wd2 = torch.from_numpy(w1).cuda(), torch.from_numpy(w2).cuda()
    r1 = build_mask("tw2", masks.img2col_forward([wd1]), 50.0, 128)       # prunes output channels of layer 1 too
    r2 = build_mask("tw1", masks.img2col_forward([wd2]), 60.0, 128)
    l1, l2 = ConvTWLayer(wd1, r1.tiles[0], dt), ConvTWLayer(wd2, r2.tiles[0], dt)
    xd = torch.from_numpy(x).to(dt).cuda()
    planes1, geo = l1.pack_input(xd)
    ct1 = l1.masked_conv(planes1, geo, activation="relu")
    planes2, geo2 = l2.repack_input(ct1, geo)
    y = l2.unpack_output(l2.masked_conv(planes2, geo2), geo2).float().cpu().numpy()
    # oracle: layer 1 in float32 on the 16-bit inputs, rounded to 16 bit as the GPU stores it, then layer 2
    x16 = xd.float().cpu().numpy()
    a1 = og.masked_matmul_dense(og.im2col_nhwc(x16, kh, kw), wd1.to(dt).float().cpu().numpy().reshape(-1, c1),
                                r1.masks[0].cpu().numpy())
    a1 = np.maximum(a1, 0).astype(np.float16).astype(np.float32).reshape(B, H, W, c1)
    # the GPU's own layer-1 output must be that, up to the last bit of the 16-bit rounding
    got1 = l1.unpack_output(ct1, geo).float().cpu().numpy()
    assert og.max_rel_error(got1, a1) <= 1e-2
    ref = og.masked_matmul_dense(og.im2col_nhwc(got1, kh, kw), wd2.to(dt).float().cpu().numpy().reshape(-1, c2),
                                 r2.masks[0].cpu().numpy()).reshape(B, H, W, c2)
    assert og.max_rel_error(y, ref) <= 1e-2
    assert og.elementwise_violations(y, ref, rtol=1e-2, floor=1e-3) == 0
    l1.close()
    l2.close()


def test_convolution_with_split_k_units():
    """One 128-channel output tile that keeps 3456 of its 4608 kernel rows: 54 K blocks on a machine with
    SMs to spare, so the scheduler cuts the tile's kept rows into ranges (split-K) and a second kernel
    adds the partial sums up; with bias and ReLU in the epilogue, against the oracle and against the same
    layer with split-K turned off."""
    import ctypes as C
    from tilesparsity_b200 import ConvTWLayer, _lib
    from tilesparsity_b200.tiles import tiles_from_lists
    g = synth.rng(77)
    B, H, W, cin, cout, kh, kw = 16, 14, 14, 512, 128, 3, 3
    K = kh * kw * cin
    x = np.maximum(g.standard_normal((B, H, W, cin), dtype=np.float32), 0)
    w = (g.standard_normal((kh, kw, cin, cout), dtype=np.float32) * np.float32(np.sqrt(2.0 / K))).astype(np.float32)
    rows = np.sort(g.permutation(K)[:3456]).astype(np.int32)
    ts = tiles_from_lists(K, cout, 128, [rows])
    wd = torch.from_numpy(w).cuda()
    layer = ConvTWLayer(wd, ts, torch.bfloat16)
    xd = torch.from_numpy(x).to(torch.bfloat16).cuda()
    from tilesparsity_b200.conv import geometry
    geo = geometry(B, H, W, kh, kw)
    parts = np.zeros(1, np.int32)
    p32 = lambda a: a.ctypes.data_as(C.POINTER(C.c_int32))
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    _lib.check(_lib.lib.ts_plan_split(1, p32(np.array([3456], np.int32)), p32(np.array([128], np.int32)), kw * cin,
                                      int(geo["m_padded"]), sms, p32(parts)))
    assert parts[0] > 1, "the case is meant to exercise split units"
    bias = torch.from_numpy(g.standard_normal(cout, dtype=np.float32)).cuda()
    y = layer.forward(xd, bias=bias, activation="relu")
    layer.layer.check()
    mask = np.zeros((K, cout), bool)
    mask[rows] = True
    x16 = xd.float().cpu().numpy()
    w16 = wd.to(torch.bfloat16).float().cpu().numpy().reshape(-1, cout)
    ref = og.masked_matmul_dense(og.im2col_nhwc(x16, kh, kw), w16, mask).reshape(B, H, W, cout)
    ref = np.maximum(ref + bias.cpu().numpy(), 0.0)
    out = y.float().cpu().numpy()
    assert og.max_rel_error(out, ref) <= 1e-2
    assert og.elementwise_violations(out, ref, rtol=1e-2, floor=1e-3) == 0
    layer.layer.set_split_k(False)
    y2 = layer.forward(xd, bias=bias, activation="relu")
    assert og.max_rel_error(y2.float().cpu().numpy(), out) <= 4e-3
    layer.close()
