"""Host-side logic and the C-ABI surface, without a GPU."""
import ctypes as C
import os
import re

import numpy as np
import pytest

from tilesparsity_b200 import _lib, synth
from tilesparsity_b200.tiles import (mask_to_offsets, offsets_to_indices, reference_partition,
                                     tile_bounds_from_col_mask, tiles_from_lists, tiles_from_mask)

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    hdr = open(os.path.join(ROOT, "include", "tilesparse.h")).read()
    hdr = re.sub(r"/\*.*?\*/", "", hdr, flags=re.S)
    names = set(re.findall(r"\b(ts_[a-z0-9_]+)\s*\(", hdr))
    assert len(names) >= 20
    for n in sorted(names):
        assert hasattr(_lib.lib, n), f"{n} is declared in tilesparse.h but not exported"
        assert n in _lib.SIGNATURES, f"{n} has no ctypes signature"
    assert _lib.lib.ts_version() >= 100


def test_compute_entry_points_fail_loudly_without_a_gpu():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    h = C.c_void_p()
    rc = _lib.lib.ts_layer_create(C.byref(h), 64, 128, 128, _lib.TS_DTYPE_F16)
    assert rc == _lib.TS_ERR_CUDA and "failed" in _lib.last_error()
    from tilesparsity_b200 import build_mask
    with pytest.raises(RuntimeError):
        build_mask("tw1", [np.ones((8, 8), np.float32)], 50.0)


def test_argument_validation_needs_no_gpu():
    h = C.c_void_p()
    assert _lib.lib.ts_layer_create(C.byref(h), 0, 128, 128, 0) == _lib.TS_ERR_INVALID
    assert _lib.lib.ts_layer_create(C.byref(h), 8, 8, 200, 0) == _lib.TS_ERR_INVALID
    assert _lib.lib.ts_layer_create(C.byref(h), 8, 8, 128, 2) == _lib.TS_ERR_INVALID
    assert "dtype" in _lib.last_error()
    assert _lib.lib.ts_masked_gemm(None, 8, None, 8, None, 8, 1.0, 0.0, None) == _lib.TS_ERR_INVALID
    assert _lib.lib.ts_build_tw_mask(99, 1, None, None, None, None, 128, 50.0, 0, 0.0, None, None, None,
                                     C.byref(h), None) == _lib.TS_ERR_INVALID
    assert _lib.lib.ts_build_pattern_mask(7, 1, None, None, None, None, 50.0, None, None, None, None) == _lib.TS_ERR_INVALID
    assert "pattern" in _lib.last_error()
    assert _lib.lib.ts_build_pattern_mask(0, 0, None, None, None, None, 50.0, None, None, None, None) == _lib.TS_ERR_INVALID
    assert _lib.lib.ts_masked_gemm_host_async(None, 8, None, None, 1.0, 0.0, None) == _lib.TS_ERR_INVALID
    assert _lib.lib.ts_masked_gemm_host_wait(None, None) == _lib.TS_ERR_INVALID


def test_pruning_fun_dispatch_matches_the_reference_names():
    from tilesparsity_b200 import masks
    for name in ("tw1", "tw2", "tw1m", "tw2m", "ew", "vw", "bw"):
        assert callable(masks.pruning_fun(name))
    with pytest.raises(KeyError):
        masks.pruning_fun("tw3")


def test_shard_plan_is_lpt_and_balanced():
    cost = np.array([5, 3, 8, 1, 7, 2], dtype=np.int64)
    own = np.zeros(6, dtype=np.int32)
    rc = _lib.lib.ts_shard_plan(6, cost.ctypes.data_as(C.POINTER(C.c_int64)), 2, own.ctypes.data_as(C.POINTER(C.c_int32)))
    assert rc == 0
    loads = [int(cost[own == p].sum()) for p in range(2)]
    assert sorted(loads) == [13, 13]
    g = synth.rng(1)
    cost = g.integers(1, 4096, 128).astype(np.int64)
    own = np.zeros(128, dtype=np.int32)
    _lib.lib.ts_shard_plan(128, cost.ctypes.data_as(C.POINTER(C.c_int64)), 8, own.ctypes.data_as(C.POINTER(C.c_int32)))
    loads = np.array([cost[own == p].sum() for p in range(8)])
    assert loads.max() <= loads.mean() * 1.02


def test_offsets_round_trip_and_reference_partition():
    m = np.array([0, 1, 1, 0, 1, 0, 0, 1])
    off = mask_to_offsets(m)
    assert off.tolist() == [1, 1, 2, 4]                    # index minus position
    assert offsets_to_indices(off).tolist() == [1, 2, 4, 7]
    n_ori, n_cal = reference_partition(768, 384, 128)      # the README's 50 % x 50 % case
    assert n_ori == [256, 256, 256] and n_cal == [128, 128, 128]
    n_ori, n_cal = reference_partition(3072, 1000, 128)
    assert sum(n_ori) == 3072 and sum(n_cal) == 1000 and n_cal[-1] == 1000 - 7 * 128


def test_tile_bounds_follow_the_regrouping_rule():
    assert tile_bounds_from_col_mask(np.ones(300, bool), 128).tolist() == [0, 128, 256, 300]
    assert tile_bounds_from_col_mask(np.ones(256, bool), 128).tolist() == [0, 128, 256]   # no cut at the edge
    cm = np.zeros(20, bool)
    cm[[1, 3, 4, 9, 10, 11, 18]] = True
    assert tile_bounds_from_col_mask(cm, 3).tolist() == [0, 5, 12, 20]                    # cut right after the 3rd kept column
    assert tile_bounds_from_col_mask(np.zeros(10, bool), 4).tolist() == [0, 10]


def test_tiles_from_mask_and_back():
    g = synth.rng(2)
    cm = g.random(400) < 0.6
    nt = len(tile_bounds_from_col_mask(cm, 64)) - 1
    ts = tiles_from_lists(50, 400, 64, synth.random_kept_lists(50, nt, 10, 4), cm)
    mask = ts.dense_mask()
    back = tiles_from_mask(mask, 64, cm)
    assert back.kept_k.tolist() == ts.kept_k.tolist() and back.kept_n.tolist() == ts.kept_n.tolist()
    assert np.array_equal(ts.relative_k() + np.concatenate([np.arange(10)] * nt), ts.kept_k)
    bad = mask.copy()
    bad[0, np.flatnonzero(cm)[0]] ^= True
    with pytest.raises(ValueError):
        tiles_from_mask(bad, 64, cm)
    with pytest.raises(ValueError):
        tiles_from_lists(50, 400, 64, [np.array([3, 2])] * nt, cm)
    assert ts.kept_flops_per_row() == 2 * int((ts.k_counts() * ts.n_counts()).sum())


def test_img2col_round_trip_on_the_host():
    """img2col_forward / img2col_back_ward (Pruning/VGG/prune_algo.py:16-37): HWIO kernels become
    [(kh*kw*cin), cout] matrices of absolute values with row index (kh*KW + kw)*cin_total + cin, 2-D
    weights pass through, and masks go back to the shapes of the weights they belong to."""
    import torch
    from tilesparsity_b200 import masks
    g = synth.rng(1)
    conv = g.standard_normal((3, 3, 8, 16)).astype(np.float32)
    fc = g.standard_normal((32, 10)).astype(np.float32)
    two_d = masks.img2col_forward([conv, fc])
    assert tuple(two_d[0].shape) == (72, 16) and tuple(two_d[1].shape) == (32, 10)
    assert float(two_d[0][(1 * 3 + 2) * 8 + 5, 7]) == abs(float(conv[1, 2, 5, 7]))
    assert np.array_equal(two_d[1].numpy(), np.abs(fc))
    m = [(t > 0.5) for t in two_d]
    back = masks.img2col_back_ward(m, [conv, fc])
    assert tuple(back[0].shape) == conv.shape and tuple(back[1].shape) == fc.shape
    assert bool(back[0][1, 2, 5, 7]) == bool(abs(conv[1, 2, 5, 7]) > 0.5)
    assert torch.equal(back[0].reshape(72, 16), m[0])
    with pytest.raises(ValueError):
        masks.img2col_back_ward([m[1]], [conv])
