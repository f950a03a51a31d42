"""The allocation-free tw1 row stage (ts_tw1_row_keep_noalloc) against ts_build_tw_mask.

Some users of this library cannot call cudaMalloc while they run (a plugin inside a framework that
owns the device heap, a server with a memory budget fixed at start-up).  For them the library has
one entry point whose scratch is a fixed array inside the library.  Because that array is shared by
every call and keeps the previous call's contents, the check runs two calls in a row on different
inputs: each must equal what the allocating entry point produces for the same input, bit for bit.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _expected_flags(scores_np, sparsity, G):
    from tilesparsity_b200 import build_mask
    res = build_mask("tw1", [scores_np], sparsity, G)
    ts = res.tiles[0]
    flags = np.zeros((ts.n_tiles, ts.K), dtype=np.uint8)
    for t in range(ts.n_tiles):
        flags[t, ts.tile_rows(t)] = 1
    return flags, res.thresholds[1]


def test_two_calls_in_a_row_match_the_allocating_entry_point():
    from tilesparsity_b200 import masks as tm
    g = np.random.Generator(np.random.PCG64(2024))
    first = np.abs(g.standard_normal((768, 3072), dtype=np.float32) * np.float32(0.02))
    second = np.abs(g.standard_normal((300, 1000), dtype=np.float32))          # other shape, ragged last tile
    for call, (scores, sparsity, G) in enumerate([(first, 75.0, 128), (second, np.float64(40.0), 128),
                                                  (first, 90.0, 64)]):
        want, want_thr = _expected_flags(scores, sparsity, G)
        dev = torch.from_numpy(scores).cuda()
        out = torch.full(want.shape, 255, dtype=torch.uint8, device="cuda")    # caller-owned output
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        got, thr = tm.tw1_row_keep_noalloc(dev, sparsity, G, out=out)
        torch.cuda.synchronize()
        free_after = torch.cuda.mem_get_info()[0]
        assert got.data_ptr() == out.data_ptr()
        assert np.array_equal(got.cpu().numpy(), want)
        assert thr == want_thr
        # The property the entry point exists for: the device's free memory is the same after the call
        # as before it.  (The very first call of a process may still load the kernels' code.)
        if call > 0:
            assert free_after == free_before, f"call {call} changed free device memory by {free_before - free_after} bytes"


def test_inputs_beyond_the_built_in_scratch_are_rejected():
    from tilesparsity_b200 import TileSparseError
    from tilesparsity_b200 import masks as tm
    big = torch.zeros((4096, 257 * 128), dtype=torch.float32, device="cuda")   # 257 tiles x 4096 rows > 2**20
    with pytest.raises(TileSparseError) as e:
        tm.tw1_row_keep_noalloc(big, 50.0, 128)
    assert e.value.code == 4 and "exceed" in str(e.value)
