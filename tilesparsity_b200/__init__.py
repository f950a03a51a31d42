"""tilesparsity_b200: B200-native Stream Masked GEMM and tile-wise mask construction.

The compute path is libtilesparse.so (hand-written sm_100a CUDA behind a C ABI, see
include/tilesparse.h); this package is the host-side mirror of the reference's operator surface.
Importing it requires the built library: `python tilesparsity_b200/build.py`.
"""
from . import tiles  # noqa: F401  (pure NumPy, always importable)
from ._lib import TileSparseError, lib  # noqa: F401
from .layer import TEWLayer, TWLayer, masked_linear, masked_matmul, transpose16  # noqa: F401
from .masks import MaskResult, build_mask, pruning_fun  # noqa: F401,E402
