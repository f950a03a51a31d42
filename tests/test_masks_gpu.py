"""GPU mask builder vs the reference's masks (golden fixtures) and the CPU oracle: bit-exact."""
import numpy as np
import pytest
import torch

from make_golden import BERT_CASES, CASES, case_inputs, load_golden
from oracle import tw_masks as om

pytestmark = pytest.mark.gpu


def _gpu_masks(algo, scores, sparsity, gran, g1):
    from tilesparsity_b200 import masks as tm
    return tm.build_mask(algo, scores, sparsity, gran, g1, want_residual=algo.endswith("m"))


TILE_CASES = sorted(n for n in CASES if CASES[n][0] not in ("ew", "vw", "bw"))
BW_CASES = sorted(n for n in CASES if CASES[n][0] == "bw")
PATTERN_CASES = sorted(n for n in CASES if CASES[n][0] in ("ew", "vw"))


@pytest.mark.parametrize("name", PATTERN_CASES)
def test_pattern_masks_match_reference_golden(name):
    """Element-wise and vector-wise baselines: bit for bit the reference's masks, through the same
    pruning_fun(name)(scores, sparsity) call the reference's hooks make."""
    from tilesparsity_b200 import masks as tm
    algo, shapes, sparsity, _, _, _, _ = CASES[name]
    scores = case_inputs(name)
    got = tm.pruning_fun(algo)(scores, sparsity)
    gold = load_golden(name)
    assert len(got) == len(gold)
    for m, g in zip(got, gold):
        assert m.shape == g.shape
        assert m.dtype == (np.float64 if algo == "vw" else np.bool_)
        assert np.array_equal(m.astype(bool), g), f"{name}: {int((m.astype(bool) != g).sum())} mask bits differ"


@pytest.mark.parametrize("algo,sparsity,shapes,seed", [
    ("ew", 75.0, [(256, 1024)], 71), ("ew", 33.3, [(100, 257), (64, 96)], 72), ("ew", 0.0, [(32, 48)], 73),
    ("ew", 100.0, [(32, 48)], 74), ("vw", 75.0, [(256, 1024)], 75), ("vw", 87.5, [(100, 257)], 76),
    ("vw", 10.0, [(40, 64)], 77), ("vw", 50.0, [(5, 33)], 78),
])
def test_pattern_masks_match_oracle(algo, sparsity, shapes, seed):
    from tilesparsity_b200 import masks as tm
    g = np.random.Generator(np.random.PCG64(seed))
    scores = [np.abs(g.standard_normal(s, dtype=np.float32)) for s in shapes]
    scores[0][:3, :5] = scores[0][0, 0]              # duplicates around the ranks
    ref = om.pruning_fun(algo)(scores, sparsity)
    got, thr = tm.build_pattern_mask(algo, scores, sparsity)
    for a, b in zip(got, ref):
        assert np.array_equal(a.cpu().numpy(), np.asarray(b).astype(bool))
    if algo == "ew":
        flat = np.concatenate([s.reshape(-1).astype(np.float64) for s in scores])
        assert thr == float(np.percentile(flat, sparsity))


@pytest.mark.parametrize("name", TILE_CASES)
def test_matches_reference_golden(name):
    algo, shapes, sparsity, gran, g1, seed, dist = CASES[name]
    scores = case_inputs(name)
    res = _gpu_masks(algo, scores, sparsity, gran, g1)
    gold = load_golden(name)
    assert len(res.masks) == len(gold)
    for m, g in zip(res.masks, gold):
        got = m.cpu().numpy()
        assert got.shape == g.shape
        assert np.array_equal(got, g), f"{name}: {int((got != g).sum())} mask bits differ from the reference"


@pytest.mark.parametrize("name", TILE_CASES)
def test_tile_lists_describe_the_mask(name):
    algo, shapes, sparsity, gran, g1, seed, dist = CASES[name]
    scores = case_inputs(name)
    res = _gpu_masks(algo, scores, sparsity, gran, g1)
    for i, (m, ts) in enumerate(zip(res.masks, res.tiles)):
        tw = ts.dense_mask()
        full = m.cpu().numpy()
        if res.residuals is not None:
            r = res.residuals[i].cpu().numpy()
            assert not (r & tw).any()
            assert np.array_equal(tw | r, full)
        else:
            assert np.array_equal(tw, full)
        for t in range(ts.n_tiles):
            rows = ts.tile_rows(t)
            assert np.all(np.diff(rows) > 0)


@pytest.mark.parametrize("algo,sparsity,gran,g1,shapes,seed", [
    ("tw1", 75.0, 128, None, [(256, 1024)], 1),
    ("tw1", np.float64(62.5), 128, None, [(128, 384), (96, 640)], 2),
    ("tw1", 33.3, 64, None, [(200, 333)], 3),
    ("tw2", 75.0, 128, None, [(256, 1024)], 4),
    ("tw2", 90, 128, None, [(192, 2048)], 5),
    ("tw2", 40.0, 32, None, [(100, 257), (64, 96)], 6),
    ("tw1m", 75.0, 128, 1.5, [(256, 1024)], 7),
    ("tw2m", 60.0, 64, 2.0, [(160, 512)], 8),
])
def test_matches_oracle(algo, sparsity, gran, g1, shapes, seed):
    g = np.random.Generator(np.random.PCG64(seed))
    scores = [np.abs(g.standard_normal(s, dtype=np.float32) * np.float32(0.05)) for s in shapes]
    fn = om.pruning_fun(algo)
    ref = fn(scores, sparsity, gran) if g1 is None else fn(scores, sparsity, gran, g1)
    res = _gpu_masks(algo, scores, sparsity, gran, g1)
    for m, r in zip(res.masks, ref):
        assert np.array_equal(m.cpu().numpy(), np.asarray(r, dtype=bool))


@pytest.mark.parametrize("name", sorted(BERT_CASES))
def test_bert_types_match_reference_golden(name):
    """Pruning types 2, 7 and 8 against the masks of the reference's own MyHook.py: bit for bit."""
    ptype, shapes, sparsity, gran, seed, dist = BERT_CASES[name]
    scores = case_inputs(name)
    gold = load_golden(name)
    mode = {2: "bert_type2", 7: "bert_type7", 8: "bert_type8"}[ptype]
    if ptype == 2:
        got = [_gpu_masks(mode, [sc], sparsity, gran, None).masks[0] for sc in scores]
    else:
        got = _gpu_masks(mode, scores, sparsity, gran, None).masks
    assert len(got) == len(gold)
    for m, g in zip(got, gold):
        m = m.cpu().numpy()
        assert m.shape == g.shape
        assert np.array_equal(m, g), f"{name}: {int((m != g).sum())} mask bits differ from the reference"


def test_bert_variants_and_topk():
    g = np.random.Generator(np.random.PCG64(77))
    s = np.abs(g.standard_normal((192, 512), dtype=np.float32))
    for name, ref in [("bert_type7", om.bert_type7([s], 70.0, 128)[0]), ("bert_type8", om.bert_type8([s], 50.0, 128)[0]),
                      ("bert_type2", om.bert_type2(s, 75.0, 128)), ("topk_l1", om.topk_l1(s, 75.0, 128))]:
        sp = {"bert_type7": 70.0, "bert_type8": 50.0}.get(name, 75.0)
        res = _gpu_masks(name, [s], sp, 128, None)
        assert np.array_equal(res.masks[0].cpu().numpy(), np.asarray(ref, dtype=bool)), name
    # ties: equal rows must be resolved towards the lower index
    t = np.ones((64, 128), dtype=np.float32)
    res = _gpu_masks("topk_l1", [t], 75.0, 128, None)
    assert np.array_equal(res.tiles[0].tile_rows(0), np.arange(16))


@pytest.mark.parametrize("n,q", [(1, 50.0), (2, 75.0), (1000, 75.0), (4097, 33.3), (100003, np.float64(12.5)),
                                 (65536, 100.0), (65536, 0.0), (3000000, 98.5)])
def test_percentile_matches_numpy(n, q):
    from tilesparsity_b200 import masks as tm
    g = np.random.Generator(np.random.PCG64(n))
    v = (g.standard_normal(n, dtype=np.float32) * np.float32(3.0)).astype(np.float32)
    v[: n // 7] = v[0]                    # duplicates around the ranks
    ref = np.percentile([np.float32(x) for x in v] if n <= 5000 else v, q)
    got = tm.percentile(torch.from_numpy(v).cuda(), q)
    assert float(ref) == got


def test_conv_kernel_masks_round_trip_through_pruning_fun():
    """The hooks' call sequence (Pruning/VGG/myhook.py:199-209): img2col_forward, pruning_fun, then
    img2col_back_ward hands 4-D HWIO masks back; checked against the reference's golden tw2 mask of a
    3 x 3 x 32 x 160 kernel."""
    from tilesparsity_b200 import masks as tm
    algo, shapes, sparsity, gran, g1, seed, dist = CASES["tw2_conv"]
    g = np.random.Generator(np.random.PCG64(seed))
    w = (g.standard_normal(shapes[0], dtype=np.float32) * np.float32(np.sqrt(2.0 / np.prod(shapes[0][:-1])))).astype(np.float32)
    scores = [t.numpy() for t in tm.img2col_forward([w])]
    assert np.array_equal(scores[0], case_inputs("tw2_conv")[0])
    masks2d = tm.pruning_fun(algo)(scores, sparsity, gran)
    masks4d = tm.img2col_back_ward(masks2d, [w])
    assert masks4d[0].shape == w.shape
    assert np.array_equal(masks4d[0].reshape(-1, w.shape[3]), load_golden("tw2_conv")[0])


def test_taylor_scores_accumulate_on_the_device_and_prune_like_the_reference():
    """square(dL/dmask * w) per step in float32, summed in float64 on the GPU, equals the NumPy
    accumulation bit for bit; pruning from it equals the reference's masks for the same scores."""
    from make_golden import taylor_steps
    from tilesparsity_b200 import masks as tm
    algo, shapes, sparsity, gran, g1, seed, dist = CASES["tw1_taylor64_grp"]
    g = np.random.Generator(np.random.PCG64(seed))
    layers = [taylor_steps(g, shp) for shp in shapes]            # ((w, grads), acc) per layer, in case order
    weights = [torch.from_numpy(w).cuda() for (w, _), _ in layers]
    ts = tm.TaylorScores(weights)
    for step in range(3):
        ts.accumulate([torch.from_numpy(grads[step]).cuda() for (_, grads), _ in layers], weights)
    for a, (_, acc) in zip(ts.acc, layers):
        assert np.array_equal(a.cpu().numpy(), acc)
    masks, res = ts.prune("tw1", sparsity, gran)
    gold = load_golden("tw1_taylor64_grp")
    for m, gmask, shp in zip(masks, gold, shapes):
        assert tuple(m.shape) == tuple(shp)
        assert np.array_equal(m.cpu().numpy().reshape(gmask.shape), gmask)
    assert all(float(a.abs().sum()) == 0.0 for a in ts.acc)       # cleared after pruning, as the hook does
    with pytest.raises(ValueError):
        tm.build_mask("tw2", [np.ones((8, 8))], 50.0)             # float64 scores: tw1 / type 7 only


@pytest.mark.parametrize("name", BW_CASES)
def test_block_wise_masks_match_reference_golden_up_to_threshold_ties(name):
    """The reference's block norms come out of the host's BLAS (np.linalg.norm of a 2-D slice), so a
    block may differ from the stored mask only if its norm lies within 1e-6 (relative) of the
    threshold; every other block must match, and in these cases none differs at all."""
    from tilesparsity_b200 import masks as tm
    algo, shapes, sparsity, _, _, _, _ = CASES[name]
    scores = case_inputs(name)
    got = tm.pruning_fun("bw")(scores, sparsity)
    gold = load_golden(name)
    _, exact, thr = om.bw(scores, sparsity, return_norms=True)
    near = np.abs(exact - thr) <= 1e-6 * abs(thr)
    idx = 0
    for m, g, s in zip(got, gold, scores):
        assert m.dtype == np.float64 and m.shape == g.shape
        for i in range(0, s.shape[0], 32):
            for j in range(0, s.shape[1], 32):
                a, b = m[i:i + 32, j:j + 32].astype(bool), g[i:i + 32, j:j + 32]
                assert a.all() or not a.any()
                assert np.array_equal(a, b) or near[idx], f"{name}: block ({i}, {j}) differs away from the threshold"
                idx += 1
