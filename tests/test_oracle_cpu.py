"""The CPU oracle against the reference's own outputs (golden fixtures) and against NumPy."""
import numpy as np
import pytest

from make_golden import BERT_CASES, CASES, case_inputs, load_golden
from oracle import masked_gemm as og
from oracle import tw_masks as om
from tilesparsity_b200 import synth
from tilesparsity_b200.tiles import tiles_from_lists, tiles_from_mask


@pytest.mark.parametrize("name", sorted(CASES))
def test_oracle_reproduces_reference_masks(name):
    algo, shapes, sparsity, gran, g1, seed, dist = CASES[name]
    scores = case_inputs(name)
    fn = om.pruning_fun(algo)
    if gran is None:
        mine = fn(scores, sparsity)
    else:
        mine = fn(scores, sparsity, gran) if g1 is None else fn(scores, sparsity, gran, g1)
    gold = load_golden(name)
    assert len(mine) == len(gold)
    for a, b in zip(mine, gold):
        assert np.array_equal(np.asarray(a, dtype=bool), b)


@pytest.mark.parametrize("name", sorted(BERT_CASES))
def test_oracle_reproduces_reference_bert_masks(name):
    """Masks of the reference's own Pruning/BERT/utils/MyHook.py (types 2, 7, 8), stored by make_golden."""
    ptype, shapes, sparsity, gran, seed, dist = BERT_CASES[name]
    scores = case_inputs(name)
    if ptype == 2:
        mine = [om.bert_type2(sc, sparsity, gran) for sc in scores]
    else:
        mine = (om.bert_type7 if ptype == 7 else om.bert_type8)(scores, sparsity, gran)
    gold = load_golden(name)
    assert len(mine) == len(gold)
    for a, b in zip(mine, gold):
        assert np.array_equal(np.asarray(a, dtype=bool), b)


def test_bert_type7_and_type8_equal_the_pinned_algorithms():
    g = synth.rng(5)
    s = [np.abs(g.standard_normal((96, 256), dtype=np.float32)), np.abs(g.standard_normal((64, 384), dtype=np.float32))]
    for a, b in zip(om.bert_type7(s, 60.0, 128), om.tw1(s, 60.0, 128)):
        assert np.array_equal(a, b)
    # type 8 is tw2 at an un-remapped sparsity: remapping q -> 100 - sqrt(10000 - 100 q) maps 75 to 50
    a = om.bert_type8(s, np.float64(50.0), 128)
    b = om.tw2(s, 75.0, 128)
    for x, y in zip(a, b):
        assert np.array_equal(x, y)
    with pytest.raises(ValueError):
        om.bert_type7([s[0][:, :200]], 50.0, 128)


@pytest.mark.parametrize("w", [1, 3, 7, 8, 9, 15, 16, 17, 64, 96, 127, 128, 129, 130, 136, 200, 257, 333, 1000, 1280])
def test_row_norm_restatement_is_numpy_bit_for_bit(w):
    g = synth.rng(w)
    x = g.standard_normal((5, w + 3)).astype(np.float32)[:, 1:1 + w]      # a strided view, as np.split yields
    assert np.array_equal(om.norm_rows_exact(x).view(np.uint32), np.linalg.norm(x, axis=1).view(np.uint32))


@pytest.mark.parametrize("K", [1, 2, 8, 9, 129, 768])
def test_col_norm_restatement_is_numpy_bit_for_bit(K):
    x = synth.rng(K).standard_normal((K, 19)).astype(np.float32)
    assert np.array_equal(om.norm_cols_exact(x).view(np.uint32), np.linalg.norm(x, axis=0).view(np.uint32))


@pytest.mark.parametrize("n", [1, 2, 3, 10, 101, 1000, 4097])
@pytest.mark.parametrize("q", [0.0, 12.5, 33.3, 50, 75.0, 99.9, 100.0, np.float64(75.0), np.float64(41.7),
                               100 - np.sqrt(10000 - 75 * 100)])
def test_percentile_restatement_is_numpy_bit_for_bit(n, q):
    v = [np.float32(x) for x in synth.rng(n).standard_normal(n)]
    ref = np.percentile(v, q)
    got, pi, ni = om.percentile_exact(v, q)
    assert type(ref) is type(got) or ref.dtype == got.dtype
    assert ref == got and 0 <= pi <= ni < n


def test_masked_gemm_forms_agree():
    g = synth.rng(3)
    K, N, M = 96, 300, 40
    A = g.standard_normal((M, K)).astype(np.float32)
    W = g.standard_normal((K, N)).astype(np.float32)
    col = g.random(N) < 0.7
    from tilesparsity_b200.tiles import tile_bounds_from_col_mask
    nt = len(tile_bounds_from_col_mask(col, 128)) - 1
    ts = tiles_from_lists(K, N, 128, synth.random_kept_lists(K, nt, 24, 9), col)
    mask = ts.dense_mask()
    dense = og.masked_matmul_dense(A, W, mask)
    comp = og.masked_matmul_compacted(A.T.copy(), W, ts).T
    ref64 = A.astype(np.float64) @ (W.astype(np.float64) * mask)
    assert og.max_rel_error(dense, ref64) < 1e-5 and og.max_rel_error(comp, ref64) < 1e-5
    assert og.checkout_errors(comp, dense, 1e-3) == 0
    # beta / alpha
    C0 = g.standard_normal((N, M)).astype(np.float32)
    out = og.masked_matmul_compacted(A.T.copy(), W, ts, alpha=0.5, beta=2.0, Ct=C0)
    kept = ts.col_mask()
    assert np.allclose(out[kept], 0.5 * dense.T[kept] + 2.0 * C0[kept], atol=1e-4)
    assert np.array_equal(out[~kept], C0[~kept])
    # packing
    wp = og.pack_weights(W, ts)
    for t in range(ts.n_tiles):
        r, c = ts.tile_rows(t), ts.tile_cols(t)
        assert np.array_equal(wp[t * 128:t * 128 + len(c), :len(r)], W[np.ix_(r, c)].T)
    assert tiles_from_mask(mask, 128, col).kept_k.tolist() == ts.kept_k.tolist()
