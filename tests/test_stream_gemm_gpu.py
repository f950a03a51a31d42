"""The perf-driver clone and the reference-signature entry point."""
import io

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("args", [(512, 768, 768, 384, 384), (1000, 768, 3072, 384, 1536), (256, 3072, 768, 1000, 100)])
def test_driver_cross_checks_pass(args):
    from tilesparsity_b200 import stream_gemm
    buf = io.StringIO()
    r = stream_gemm.run(*args, iters=3, out=buf)
    lines = buf.getvalue().strip().splitlines()
    assert [l.split(":")[0].strip() for l in lines] == ["CUTLASS GEMM", "CUTLASS GEMM", "Stream  GEMM"]
    assert r["errors"] == [0, 0, 0]
    assert r["M"] % 8 == 0 and r["block_num"] == (r["N_pruned"] + 127) // 128


def test_cli_exit_codes():
    from tilesparsity_b200 import stream_gemm
    assert stream_gemm.main(["256", "256", "256", "128", "64", "--iters", "2"]) == 0
    assert stream_gemm.main(["256", "256", "256", "512", "64", "--iters", "2"]) == -1     # N_pruned > N
    assert stream_gemm.main(["64", "8192", "64", "8192", "64", "--iters", "2"]) == -1     # more than 32 tiles
