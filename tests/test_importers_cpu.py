"""Readers for the reference's pickled artefacts (format per Pruning/VGG/pruning.py:580-587 and
Pruning/BERT/utils/MyHook.py:54-89), exercised on files written the way the reference writes them."""
import pickle

import numpy as np

from make_golden import case_inputs, load_golden
from tilesparsity_b200 import importers
from tilesparsity_b200.tiles import mask_to_offsets


def test_mask_pickles_round_trip(tmp_path):
    tw2 = load_golden("tw2_small")[0]
    tw1m = load_golden("tw1m_small")[0]
    conv = load_golden("tw2_conv")[0].reshape(3, 3, 32, 160)
    p = tmp_path / "masks.pkl"
    with open(p, "wb") as f:
        pickle.dump({"fc/w": tw2.astype(np.float32), "lstm/w": tw1m.astype(np.int32), "conv/w": conv.astype(np.float32)}, f)
    items = dict(importers.load_mask_pickle(str(p)))
    assert items["conv/w"].shape == (288, 160)
    ts, res = importers.tiles_from_reference_mask(items["fc/w"], 128)
    assert not res.any() and np.array_equal(ts.dense_mask(), tw2)
    assert ts.n_counts().max() <= 128
    ts, res = importers.tiles_from_reference_mask(items["lstm/w"], 128)
    assert res.any() and np.array_equal(ts.dense_mask() | res, tw1m) and not (ts.dense_mask() & res).any()
    ts, res = importers.tiles_from_reference_mask(items["conv/w"], 64)
    assert np.array_equal(ts.dense_mask() | res, items["conv/w"])


def test_bert_pruned_model_pickle(tmp_path):
    g = np.random.Generator(np.random.PCG64(5))
    K, N = 96, 256
    mi = (g.random(K) < 0.4).astype(np.float32)
    mo = (g.random(N) < 0.6).astype(np.float32)
    kernel = g.standard_normal((K, N)).astype(np.float32)
    bias = g.standard_normal(N).astype(np.float32)
    ckpt = {"bert/l0/mask-i:0": mask_to_offsets(mi), "bert/l0/mask-o:0": mask_to_offsets(mo),
            "bert/l0/kernel:0": (kernel[mi.astype(bool)].T[mo.astype(bool)]).T, "bert/l0/bias:0": bias * mo}
    p = tmp_path / "pruned_model.pkl"
    with open(p, "wb") as f:
        pickle.dump(ckpt, f, pickle.HIGHEST_PROTOCOL)
    layers = importers.load_bert_pruned_model(str(p))
    assert len(layers) == 1
    L = layers[0]
    assert np.array_equal(L["kept_in"], np.flatnonzero(mi)) and np.array_equal(L["kept_out"], np.flatnonzero(mo))
    W = importers.dense_weights_from_bert_layer(L, K, N)
    assert np.array_equal(W, kernel * mi[:, None] * mo[None, :])
    ts = importers.tiles_from_bert_layer(L, K, N, 128)
    assert np.array_equal(ts.dense_mask(), (mi[:, None] * mo[None, :]) != 0)


def test_bert_dumped_model_pickle(tmp_path):
    """The layout dump_pruned_model.py writes (Pruning/BERT/utils/dump_pruned_model.py:118-140)."""
    mask = load_golden("bert7_group")[0]                        # a type-7 mask of the reference, 96 x 256
    g = np.random.Generator(np.random.PCG64(6))
    kernel = g.standard_normal(mask.shape).astype(np.float32)
    bias = g.standard_normal(mask.shape[1]).astype(np.float32)
    scope = "bert/encoder/layer_0/intermediate/dense"
    model = {"transformer_ckpt": {
        "origin_ckpt": {scope + "/kernel:0": kernel, scope + "/bias:0": bias},
        "masked_ckpt": {scope + "/kernel:0": kernel * mask},
        "absolute_mask": {scope + "/mask-o:0": mask.astype(np.float32)}}}
    p = tmp_path / "model.pkl"
    with open(p, "wb") as f:
        pickle.dump(model, f, pickle.HIGHEST_PROTOCOL)
    layers = importers.load_bert_dumped_model(str(p))
    assert len(layers) == 1
    L = layers[0]
    assert L["name"] == scope + "/kernel:0" and np.array_equal(L["mask"], mask)
    assert np.array_equal(L["masked_kernel"], kernel * mask) and np.array_equal(L["bias"], bias)
    ts, res = importers.tiles_from_dumped_layer(L, 128)
    assert not res.any() and np.array_equal(ts.dense_mask(), mask)
    with open(p, "wb") as f:
        pickle.dump({"something": 1}, f)
    import pytest
    with pytest.raises(ValueError):
        importers.load_bert_dumped_model(str(p))
