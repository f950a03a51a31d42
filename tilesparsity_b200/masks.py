"""GPU mask construction with the reference's call shape.

`pruning_fun(name)(scores, sparsity, granularity=128[, g1percent])` mirrors
Pruning/VGG/prune_algo.py:267-278 for the tile-wise algorithms (`tw1`, `tw2`, `tw1m`, `tw2m`): a
list of 2-D score arrays in, a list of 0/1 masks of the same shapes out, one threshold shared by
the whole list.  Scores may be NumPy arrays or CUDA tensors; masks come back in kind.  All scoring,
selection and thresholding runs in libtilesparse's CUDA kernels (ts_build_tw_mask); there is no CPU
path.  `build_mask` additionally returns the tile structure (per-tile kept-row lists, kept columns)
that `TWLayer` consumes, which closes the gap the reference leaves between its mask builder and its
GEMM driver.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import numpy as np
import torch

from . import _lib
from ._lib import check, lib
from .tiles import TileSet


@dataclass
class MaskResult:
    masks: list            # uint8/bool CUDA tensors [K, N], one per layer (TW part | TEW residual)
    tiles: list            # TileSet per layer: the tile-wise part
    residuals: list        # bool CUDA tensors [K, N] with the TEW residual elements, or None
    thresholds: tuple      # (column stage, row stage, residual stage); NaN where a stage did not run


def img2col_forward(weights):
    """HWIO conv kernels -> 2-D [(kh*kw*cin), cout]; absolute values (prune_algo.py:16-24)."""
    out = []
    for w in weights:
        t = w if isinstance(w, torch.Tensor) else torch.from_numpy(np.ascontiguousarray(w))
        if t.dim() == 4:
            t = t.reshape(t.shape[0] * t.shape[1] * t.shape[2], t.shape[3])
        out.append(t.abs())
    return out


def img2col_back_ward(masks, mask_shape):
    """2-D masks -> the shapes of the weights they belong to: masks of HWIO conv kernels are reshaped
    to [kh, kw, cin, cout], 2-D ones pass through (prune_algo.py:27-37; the hooks hand the result
    back to the graph's 4-D mask placeholders, Pruning/VGG/myhook.py:205-209).  `mask_shape` holds
    the original weights (anything with a `.shape`), as in the reference."""
    out = []
    for m, w in zip(masks, mask_shape):
        shp = tuple(w.shape)
        if len(shp) == 4:
            if m.shape[0] != shp[0] * shp[1] * shp[2] or m.shape[1] != shp[3]:
                raise ValueError(f"a mask of shape {tuple(m.shape)} does not belong to a kernel of shape {shp}")
            m = m.reshape(shp)
        elif len(shp) != 2:
            raise ValueError(f"weights of shape {shp} are neither a conv kernel nor a matrix")
        out.append(m)
    return out


def _is_f64(x) -> bool:
    return isinstance(x, np.floating) and not isinstance(x, np.float32)


def build_mask(name: str, scores, sparsity, granularity: int = 128, g1percent=None, want_residual: bool = False,
               device=None) -> MaskResult:
    """Runs one of the mask algorithms on the GPU.  `name` is a reference name (tw1, tw2, tw1m, tw2m),
    a BERT pruning type (bert_type2 / bert_type7 / bert_type8), topk_l1, or tw_cols_rows (column stage
    at `g1percent` percent, tile-row stage at `sparsity` percent)."""
    if name not in _lib.MASK_MODES:
        raise KeyError(f"unknown mask algorithm {name!r}")
    if not torch.cuda.is_available():
        raise RuntimeError("build_mask needs a CUDA device (there is no CPU fallback)")
    mode = _lib.MASK_MODES[name]
    tew = name in ("tw1m", "tw2m")
    if g1percent is None:
        g1percent = {"tw1m": 5, "tw2m": 1}.get(name, 0)     # the reference's defaults (prune_algo.py:180,187)
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    sc = []
    for s in scores:
        t = s if isinstance(s, torch.Tensor) else torch.from_numpy(np.ascontiguousarray(s))
        if t.dim() != 2:
            raise ValueError("scores must be 2-D (use img2col_forward for conv kernels)")
        sc.append(t)
    # float64 scores (the reference's accumulated Taylor scores) keep their type: NumPy would do every
    # step in double, and so does the library's float64 row stage
    f64 = all(t.dtype == torch.float64 for t in sc)
    if f64 and name not in ("tw1", "bert_type7"):
        raise ValueError("float64 scores are supported by tw1 and bert_type7 only; cast them to float32 for " + name)
    sc = [t.to(device=dev, dtype=torch.float64 if f64 else torch.float32) for t in sc]
    sc = [t if t.stride(1) == 1 else t.contiguous() for t in sc]
    n = len(sc)
    masks = [torch.empty((t.shape[0], t.shape[1]), dtype=torch.uint8, device=dev) for t in sc]
    resid = [torch.zeros((t.shape[0], t.shape[1]), dtype=torch.uint8, device=dev) for t in sc] \
        if (tew and want_residual) else None
    VP = C.c_void_p * n
    IA = C.c_int * n
    LA = C.c_int64 * n
    handle = C.c_void_p()
    with torch.cuda.device(dev):
        if f64:
            check(lib.ts_build_tw_mask_f64(
                mode, n, VP(*[t.data_ptr() for t in sc]), IA(*[t.shape[0] for t in sc]), IA(*[t.shape[1] for t in sc]),
                LA(*[t.stride(0) for t in sc]), int(granularity), float(sparsity),
                VP(*[m.data_ptr() for m in masks]), LA(*[m.stride(0) for m in masks]), C.byref(handle),
                C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)))
        else:
            check(lib.ts_build_tw_mask(
                mode, n, VP(*[t.data_ptr() for t in sc]), IA(*[t.shape[0] for t in sc]), IA(*[t.shape[1] for t in sc]),
                LA(*[t.stride(0) for t in sc]), int(granularity), float(sparsity),
                int(_is_f64(sparsity) or _is_f64(g1percent)), float(g1percent), VP(*[m.data_ptr() for m in masks]),
                LA(*[m.stride(0) for m in masks]), VP(*[r.data_ptr() for r in resid]) if resid else None,
                C.byref(handle), C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)))
    try:
        tiles = []
        for l, t in enumerate(sc):
            nt, nk, nn = C.c_int(), C.c_int(), C.c_int()
            check(lib.ts_mask_result_layer(handle, l, C.byref(nt), C.byref(nk), C.byref(nn)))
            b = np.zeros(nt.value + 1, np.int32)
            kp = np.zeros(nt.value + 1, np.int32)
            npz = np.zeros(nt.value + 1, np.int32)
            kk = np.zeros(max(nk.value, 1), np.int32)
            nn_a = np.zeros(max(nn.value, 1), np.int32)
            p = lambda a: a.ctypes.data_as(C.POINTER(C.c_int32))
            check(lib.ts_mask_result_copy(handle, l, p(b), p(kp), p(kk), p(npz), p(nn_a)))
            tiles.append(TileSet(int(t.shape[0]), int(t.shape[1]), int(granularity), b, kp, kk[:nk.value], npz,
                                 nn_a[:nn.value]))
        thr = (C.c_double * 3)()
        check(lib.ts_mask_result_thresholds(handle, thr))
    finally:
        lib.ts_mask_result_destroy(handle)
    # the kernels write 0 / 1 bytes: reinterpreted, not converted
    return MaskResult([m.view(torch.bool) for m in masks], tiles,
                      [r.view(torch.bool) for r in resid] if resid else None, tuple(thr))


def build_pattern_mask(name: str, scores, sparsity, device=None):
    """The reference's baseline patterns on the GPU: "ew" (element-wise, prune_algo.py:38-53), "vw"
    (vector-wise, :196-227) and "bw" (block-wise with its default 32 x 32 blocks, :229-264).  Returns
    (list of CUDA bool masks, threshold or NaN)."""
    if name not in _lib.PATTERN_MODES:
        raise KeyError(f"unknown pattern {name!r} (ew, vw, bw)")
    if not torch.cuda.is_available():
        raise RuntimeError("build_pattern_mask needs a CUDA device (there is no CPU fallback)")
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    sc = []
    for s in scores:
        t = s if isinstance(s, torch.Tensor) else torch.from_numpy(np.ascontiguousarray(s))
        if t.dim() != 2:
            raise ValueError("scores must be 2-D (use img2col_forward for conv kernels)")
        t = t.to(device=dev, dtype=torch.float32)
        sc.append(t if t.stride(1) == 1 else t.contiguous())
    n = len(sc)
    masks = [torch.empty((t.shape[0], t.shape[1]), dtype=torch.uint8, device=dev) for t in sc]
    VP, IA, LA = C.c_void_p * n, C.c_int * n, C.c_int64 * n
    thr = C.c_double()
    with torch.cuda.device(dev):
        check(lib.ts_build_pattern_mask(
            _lib.PATTERN_MODES[name], n, VP(*[t.data_ptr() for t in sc]), IA(*[t.shape[0] for t in sc]),
            IA(*[t.shape[1] for t in sc]), LA(*[t.stride(0) for t in sc]), float(sparsity),
            VP(*[m.data_ptr() for m in masks]), LA(*[m.stride(0) for m in masks]), C.byref(thr),
            C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)))
    return [m.view(torch.bool) for m in masks], thr.value


def pruning_fun(pruning_type: str):
    """Same dispatch as the reference (prune_algo.py:267-278): the tile-wise algorithms and the
    element-wise / vector-wise / block-wise baselines.  "bw" equals the reference up to blocks whose
    norm lies within rounding distance of the threshold (its norms come out of the host's BLAS).  The
    returned function takes (scores, sparsity[, granularity][, g1percent]) and returns the masks as
    NumPy arrays when given NumPy scores (bool; float64 0/1 for "vw" and "bw", as the reference does),
    as CUDA bool tensors otherwise."""
    if pruning_type in ("ew", "vw", "bw"):
        def pattern_fn(accumulated_scores, sparsity):
            masks, _ = build_pattern_mask(pruning_type, accumulated_scores, sparsity)
            if all(isinstance(s, np.ndarray) for s in accumulated_scores):
                out = [m.cpu().numpy() for m in masks]
                return [m.astype(np.float64) for m in out] if pruning_type in ("vw", "bw") else out
            return masks
        return pattern_fn
    if pruning_type not in ("tw1", "tw2", "tw1m", "tw2m"):
        raise KeyError(f"{pruning_type!r} is not one of tw1, tw2, tw1m, tw2m, ew, vw, bw")

    def fn(accumulated_scores, sparsity, granularity=128, g1percent=None):
        res = build_mask(pruning_type, accumulated_scores, sparsity, granularity, g1percent)
        if all(isinstance(s, np.ndarray) for s in accumulated_scores):
            return [m.cpu().numpy() for m in res.masks]
        return res.masks

    return fn


class TaylorScores:
    """First-order Taylor importance scores kept on the GPU, as the reference's pruning hooks keep
    them on the host: one float64 accumulator per masked layer, `accumulate` adds a step's
    square(dL/dmask * w) (compute_taylor_score and after_run, Pruning/VGG/myhook.py:44-48,248-257),
    `prune` builds the masks from the accumulated scores and clears them (myhook.py:191-235, 259-261).

    Gradients and weights are float32 CUDA tensors of the layers' own shapes (HWIO conv kernels or
    2-D matrices); the masks come back in those shapes."""

    def __init__(self, weights):
        self.shapes = [tuple(w.shape) for w in weights]
        self.device = weights[0].device
        self.acc = [torch.zeros(s, dtype=torch.float64, device=self.device) for s in self.shapes]
        self.steps = 0

    def accumulate(self, grads, weights) -> None:
        if len(grads) != len(self.acc) or len(weights) != len(self.acc):
            raise ValueError("one gradient and one weight tensor per layer")
        with torch.cuda.device(self.device):
            for g, w, a in zip(grads, weights, self.acc):
                if g.dtype != torch.float32 or w.dtype != torch.float32 or tuple(g.shape) != tuple(a.shape) \
                        or tuple(w.shape) != tuple(a.shape) or not (g.is_contiguous() and w.is_contiguous()):
                    raise ValueError("gradients and weights must be contiguous float32 tensors of the layer's shape")
                check(lib.ts_taylor_accumulate(C.c_void_p(g.data_ptr()), C.c_void_p(w.data_ptr()), C.c_void_p(a.data_ptr()),
                                               a.numel(), C.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)))
        self.steps += 1

    def prune(self, pruning_type: str, sparsity, granularity: int = 128, layers=None, reset: bool = True):
        """Masks (bool CUDA tensors in the layers' shapes) of the layers in `layers` (default: all),
        pruned together under one threshold as the reference prunes a layer group (Pruning/VGG/
        pruning.py:392-404)."""
        layers = list(range(len(self.acc))) if layers is None else list(layers)
        scores = img2col_forward([self.acc[l] for l in layers])
        res = build_mask(pruning_type, scores, sparsity, granularity)
        out = img2col_back_ward(res.masks, [self.acc[l] for l in layers])
        if reset:
            for l in layers:
                self.acc[l].zero_()
        return out, res


def percentile(values: torch.Tensor, q) -> float:
    """np.percentile(values, q) of a float32 CUDA tensor, computed by the library's radix select."""
    v = values.reshape(-1).contiguous()
    if v.dtype != torch.float32 or not v.is_cuda:
        raise ValueError("percentile takes a float32 CUDA tensor")
    out = C.c_double()
    with torch.cuda.device(v.device):
        check(lib.ts_percentile_f32(C.c_void_p(v.data_ptr()), v.numel(), float(q), int(_is_f64(q)), C.byref(out),
                                    C.c_void_p(torch.cuda.current_stream(v.device).cuda_stream)))
    return out.value


def tw1_row_keep_noalloc(score: torch.Tensor, sparsity, granularity: int = 128, out: torch.Tensor | None = None):
    """tw1 keep flags of one matrix, [n_tiles, K] uint8, through the entry point that allocates no
    device memory (its scratch is a fixed array inside the library).  Meant for callers that cannot
    allocate while they run; `out` lets such a caller pass its own pre-allocated flags tensor.
    Returns (flags, threshold).  Inputs beyond the built-in scratch raise TileSparseError."""
    if score.dtype != torch.float32 or not score.is_cuda or score.dim() != 2 or score.stride(1) != 1:
        raise ValueError("score must be a 2-D float32 CUDA tensor with contiguous rows")
    K, N = score.shape
    n_tiles = (N + granularity - 1) // granularity
    if out is None:
        out = torch.empty((n_tiles, K), dtype=torch.uint8, device=score.device)
    if tuple(out.shape) != (n_tiles, K) or out.dtype != torch.uint8 or not out.is_contiguous() or out.device != score.device:
        raise ValueError(f"out must be a contiguous uint8 [{n_tiles}, {K}] tensor on {score.device}")
    thr = C.c_double()
    with torch.cuda.device(score.device):
        check(lib.ts_tw1_row_keep_noalloc(C.c_void_p(score.data_ptr()), score.stride(0), K, N, int(granularity),
                                          float(sparsity), int(_is_f64(sparsity)), C.c_void_p(out.data_ptr()),
                                          C.byref(thr), C.c_void_p(torch.cuda.current_stream(score.device).cuda_stream)))
    return out, thr.value
