"""tilesparsity_b200: B200-native Stream Masked GEMM and tile-wise mask construction.

The compute path is libtilesparse.so (hand-written sm_100a CUDA behind a C ABI, see
include/tilesparse.h); this package is the host-side mirror of the reference's operator surface.
Using any operator requires the built library: `python tilesparsity_b200/build.py`.

The operator names resolve on first use, so the pure-NumPy helpers (`tilesparsity_b200.tiles`,
`tilesparsity_b200.synth`) can be imported by a process that never touches the GPU library.
"""
from . import tiles  # noqa: F401  (pure NumPy, always importable)

_LAZY = {
    "TileSparseError": "_lib", "lib": "_lib",
    "TEWLayer": "layer", "TWLayer": "layer", "masked_linear": "layer", "masked_matmul": "layer",
    "transpose16": "layer", "ConvTWLayer": "conv",
    "MaskResult": "masks", "build_mask": "masks", "pruning_fun": "masks",
}


def __getattr__(name):
    if name in _LAZY:
        import importlib
        value = getattr(importlib.import_module("." + _LAZY[name], __name__), name)
        globals()[name] = value
        return value
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")


def __dir__():
    return sorted(list(globals()) + list(_LAZY))
