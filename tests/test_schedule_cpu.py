"""The work distribution of the persistent masked GEMM (ts_plan_schedule: a pure host function).

The reference runs tile t on CUDA stream t (StreamMaskedGEMM/perf/basic_nn.cu:402-427); here every
(tile, 64-row batch granule) must be covered exactly once by the units handed to at most n_ctas CTAs,
units must respect the kernel variant's width, and the modelled per-CTA load must be balanced."""
import ctypes as C

import numpy as np
import pytest

from tilesparsity_b200 import _lib, synth
from tilesparsity_b200._lib import lib


def plan(k_counts, n_counts, K, M, n_ctas=148, unit_rows=0):
    kc = np.ascontiguousarray(k_counts, dtype=np.int32)
    nc = np.ascontiguousarray(n_counts, dtype=np.int32)
    p = lambda a: a.ctypes.data_as(C.POINTER(C.c_int32))
    u, g, n = C.c_int(), C.c_int(), C.c_int()
    _lib.check(lib.ts_plan_schedule(len(kc), p(kc), p(nc), K, M, n_ctas, unit_rows, C.byref(u), C.byref(g), C.byref(n),
                                    None, 0, None))
    units = np.zeros((max(n.value, 1), 4), dtype=np.int32)
    cost = np.zeros(n_ctas, dtype=np.float32)
    _lib.check(lib.ts_plan_schedule(len(kc), p(kc), p(nc), K, M, n_ctas, unit_rows, C.byref(u), C.byref(g), C.byref(n),
                                    p(units), n.value, cost.ctypes.data_as(C.POINTER(C.c_float))))
    return u.value, g.value, units[:n.value], cost[:g.value]


def check_cover(units, k_counts, n_counts, M, unit_rows, n_ctas):
    gran = (M + 63) // 64
    cover = np.zeros((len(k_counts), gran), dtype=np.int64)
    for cta, t, m0, ml in units:
        assert 0 <= cta < n_ctas and n_counts[t] > 0
        assert m0 % 64 == 0 and ml % 64 == 0 and 0 < ml <= unit_rows and m0 + ml <= gran * 64
        cover[t, m0 // 64:(m0 + ml) // 64] += 1
    live = np.asarray(n_counts) > 0
    assert (cover[live] == 1).all() and (cover[~live] == 0).all()
    # a CTA's units come in one run per CTA (the table is written CTA by CTA)
    ctas = units[:, 0]
    assert (np.diff(ctas) >= 0).all()


BERT = {"qkv": (768, 2304, 192), "attn_out": (768, 768, 192), "ffn1": (768, 3072, 192), "ffn2": (3072, 768, 768)}


@pytest.mark.parametrize("name", sorted(BERT))
@pytest.mark.parametrize("M", [4096, 1024, 1000, 64])
def test_bert_shapes_fill_the_machine(name, M):
    K, N, keep = BERT[name]
    nt = N // 128
    kc, nc = [keep] * nt, [128] * nt
    urows, grid, units, cost = plan(kc, nc, K, M)
    check_cover(units, kc, nc, M, urows, 148)
    granules = nt * ((M + 63) // 64)
    assert grid == min(148, granules)            # every SM gets work when there is enough of it
    assert cost.max() > 0 and cost.mean() / cost.max() > 0.85


@pytest.mark.parametrize("n,unit_rows", [(4096, 0), (4096, 128), (8192, 0), (16384, 0), (16384, 256)])
def test_skewed_squares(n, unit_rows):
    """Per-tile kept-row counts ~ Beta(2,5): the contiguous partition (activations within L2) and the
    blocked list schedule (beyond) both cover everything and stay balanced."""
    nt = n // 128
    kc = synth.beta_skewed_counts(n, nt, 0.25, 5000 + int(np.log2(n)))
    nc = [128] * nt
    urows, grid, units, cost = plan(kc, nc, n, n, unit_rows=unit_rows)
    assert urows == (unit_rows or 256) and grid == 148
    check_cover(units, kc, nc, n, urows, 148)
    assert cost.mean() / cost.max() > 0.9


def test_ragged_tiles_empty_tiles_and_small_grids():
    kc = [192, 0, 300, 64, 8, 1000]
    nc = [128, 128, 100, 0, 1, 128]            # tile 3 keeps no column: it gets no unit
    for M in (8, 72, 1000, 4096):
        for n_ctas in (1, 3, 148):
            urows, grid, units, cost = plan(kc, nc, 1024, M, n_ctas)
            check_cover(units, kc, nc, M, urows, n_ctas)
            assert grid <= n_ctas
    urows, grid, units, cost = plan([0, 0], [0, 0], 64, 128)
    assert len(units) == 0


def test_unit_rows_can_be_pinned_and_bad_arguments_are_rejected():
    kc, nc = [192] * 24, [128] * 24
    for ur in (128, 256):
        urows, grid, units, cost = plan(kc, nc, 768, 4096, unit_rows=ur)
        assert urows == ur and units[:, 3].max() <= ur
    with pytest.raises(_lib.TileSparseError):
        plan(kc, nc, 768, 4096, unit_rows=192)
    with pytest.raises(_lib.TileSparseError):
        plan([5], [129], 768, 4096)
    with pytest.raises(_lib.TileSparseError):
        plan(kc, nc, 768, 0)


def plan_split(k_counts, n_counts, K, M, n_ctas=148):
    kc = np.ascontiguousarray(k_counts, dtype=np.int32)
    nc = np.ascontiguousarray(n_counts, dtype=np.int32)
    parts = np.zeros(len(kc), dtype=np.int32)
    p = lambda a: a.ctypes.data_as(C.POINTER(C.c_int32))
    _lib.check(lib.ts_plan_split(len(kc), p(kc), p(nc), K, M, n_ctas, p(parts)))
    return parts.tolist()


def test_split_k_plan_cuts_only_long_chains_with_sms_to_spare():
    """A tile is cut into K ranges only when its chain of K blocks is long and its share of the SMs is at
    least twice its number of 256-row units; the reference has no counterpart (one CUTLASS launch per
    tile, StreamMaskedGEMM/perf/basic_nn.cu:396-427)."""
    conv_rows = 3 * 512          # the planes of a 3 x 3 convolution over 512 channels that exist in memory
    # VGG conv5 with 10 % of the columns and 75 % of the rows pruned: three light tiles and a 76-column
    # tile that keeps about 4300 of 4608 rows; as a GEMM over the im2col matrix and as the convolution
    assert plan_split([130, 71, 102, 4305], [128, 128, 128, 76], 4608, 12544) == [1, 1, 1, 2]
    assert plan_split([95, 65, 26, 4422], [128, 128, 128, 76], conv_rows, 16384) == [1, 1, 1, 2]
    # one 128-column tile with all 4608 rows kept
    assert plan_split([4608], [128], 4608, 12544) == [3]
    # tw2 conv5: as a GEMM the list schedule leaves a third of the SMs idle (cut), as the convolution the
    # contiguous partition fills the machine already (whole)
    assert plan_split([2318, 4594], [128, 128], 4608, 12544) == [1, 2]
    assert plan_split([3749, 859], [128, 128], conv_rows, 16384) == [1, 1]
    assert plan_split([3661, 3251], [128, 128], conv_rows, 16384) == [1, 1]
    # BERT shapes and squares: no split
    assert plan_split([768] * 6, [128] * 6, 3072, 4096) == [1] * 6
    assert plan_split([192] * 24, [128] * 24, 768, 4096) == [1] * 24
    assert plan_split([4096] * 128, [128] * 128, 16384, 16384) == [1] * 128
    # never more than four ranges, none for an empty tile, short chains stay whole
    assert plan_split([16384], [128], 16384, 256) == [4]
    assert plan_split([4608, 4608], [128, 0], 4608, 12544) == [3, 1]
    assert plan_split([1984], [128], 4608, 12544) == [1]
