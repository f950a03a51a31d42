"""Readers for the artefacts the reference's pruning runs leave behind.

* VGG / NMT: `mask_*.pkl` / `masks.pkl`, dicts or lists of 0/1 NumPy arrays, one per pruned weight
  (Pruning/VGG/pruning.py:580-587,639-640; Pruning/NMT/nmt/train.py:741-742).  Conv kernels are HWIO
  and are viewed as [(kh*kw*cin), cout] (img2col_forward, Pruning/VGG/prune_algo.py:16-24).
* BERT: `pruned_model.pkl` written by exportPrunedModel (Pruning/BERT/utils/MyHook.py:54-89): for every
  masked dense layer four entries in order -- the input-side offsets (`...mask-i...`), the output-side
  offsets (`...mask-o...`), the compacted kernel [kept_in, kept_out] and the masked bias.  Offsets are
  "index minus position" (convert_mask_to_offset, MyHook.py:66-74).

* BERT: the `<name>.pkl` of dump_pruned_model.py (Pruning/BERT/utils/dump_pruned_model.py:118-140):
  `model["transformer_ckpt"]` with `origin_ckpt` (kernel and bias per masked dense layer),
  `masked_ckpt` (kernel * mask) and `absolute_mask` (the layer's 2-D 0/1 `mask-o` variable,
  modeling.py:992-1007), keyed by TensorFlow variable names.

Everything here is host-side format handling (NumPy only); the results are TileSets / dense masks that
`TWLayer` and `ts_layer_set_tiles` take as they are.
"""
from __future__ import annotations

import pickle

import numpy as np

from .tiles import TileSet, offsets_to_indices, tiles_from_mask


def as_2d(mask) -> np.ndarray:
    """HWIO conv masks -> [(kh*kw*cin), cout]; 2-D masks unchanged."""
    m = np.asarray(mask)
    if m.ndim == 4:
        m = m.reshape(m.shape[0] * m.shape[1] * m.shape[2], m.shape[3])
    if m.ndim != 2:
        raise ValueError(f"cannot view a mask of shape {m.shape} as a weight matrix")
    return m != 0


def load_mask_pickle(path: str):
    """A VGG/NMT mask pickle -> list of (name, bool [K, N]) in stored order."""
    with open(path, "rb") as f:
        obj = pickle.load(f)
    if isinstance(obj, dict):
        items = list(obj.items())
    else:
        items = [(str(i), m) for i, m in enumerate(obj)]
    return [(str(k), as_2d(v)) for k, v in items]


def tiles_from_reference_mask(mask, G: int = 128, strict: bool = False):
    """TileSet (tile-wise part) and residual (bool [K, N]) of a reference mask.

    The column mask is "columns that keep anything".  Tile boundaries follow the reference's rule for
    the pattern the mask was built with: `tw2` regroups the surviving columns G at a time, `tw1` uses
    fixed tiles of G columns; a mask without pruned columns is read as `tw1`.  Elements kept outside the
    rows a tile keeps in all its columns (TEW residual, or a mask that is not tile-wise at all) are
    returned as the residual; with strict=True they raise instead."""
    m = as_2d(mask)
    col_mask = m.any(axis=0)
    ts = tiles_from_mask(m, G, None if col_mask.all() else col_mask, strict=strict)
    residual = m & ~ts.dense_mask()
    return ts, residual


def load_bert_pruned_model(path: str):
    """pruned_model.pkl -> list of dicts {name, kept_in, kept_out, kernel [kept_in, kept_out], bias}.

    kept_in / kept_out are absolute ascending indices rebuilt from the stored offsets."""
    with open(path, "rb") as f:
        ckpt = pickle.load(f)
    keys = list(ckpt.keys())
    layers = []
    for i, k in enumerate(keys):
        if "mask-i" not in k:
            continue
        if i + 3 >= len(keys):
            raise ValueError(f"{k}: the pickle ends before the layer's four entries")
        mi, mo, kernel, bias = (np.asarray(ckpt[keys[i + d]]) for d in range(4))
        kept_in = offsets_to_indices(mi.astype(np.int32))
        kept_out = offsets_to_indices(mo.astype(np.int32))
        if kernel.shape != (len(kept_in), len(kept_out)):
            raise ValueError(f"{k}: compacted kernel {kernel.shape} does not match {len(kept_in)} x {len(kept_out)} offsets")
        layers.append({"name": k, "kept_in": kept_in, "kept_out": kept_out, "kernel": kernel, "bias": bias})
    return layers


def tiles_from_bert_layer(layer: dict, K: int, N: int, G: int = 128) -> TileSet:
    """One exported BERT layer as a TileSet: its kept output columns regrouped G at a time, every tile
    keeping the layer's kept input rows (the export stores one row set per layer)."""
    col_mask = np.zeros(N, dtype=bool)
    col_mask[layer["kept_out"]] = True
    from .tiles import tile_bounds_from_col_mask, tiles_from_lists
    n_tiles = len(tile_bounds_from_col_mask(col_mask, G)) - 1
    return tiles_from_lists(K, N, G, [layer["kept_in"].astype(np.int32)] * n_tiles, col_mask)


def dense_weights_from_bert_layer(layer: dict, K: int, N: int) -> np.ndarray:
    """The layer's weights scattered back to [K, N] (zeros where pruned), ready for `TWLayer.pack`."""
    W = np.zeros((K, N), dtype=np.asarray(layer["kernel"]).dtype)
    W[np.ix_(layer["kept_in"], layer["kept_out"])] = layer["kernel"]
    return W


def load_bert_dumped_model(path: str):
    """The pickle of dump_pruned_model.py -> list of dicts {name, kernel [K, N], masked_kernel, mask
    (bool [K, N]), bias or None}, one per masked dense layer, in stored order.

    Layers are matched by variable scope: `<scope>/mask-o:0` in `absolute_mask` belongs to
    `<scope>/kernel:0` (dump_pruned_model.py:52-76 reads kernel, bias, mask-o as neighbours)."""
    with open(path, "rb") as f:
        model = pickle.load(f)
    try:
        ck = model["transformer_ckpt"]
        masks, masked, origin = ck["absolute_mask"], ck["masked_ckpt"], ck.get("origin_ckpt", {})
    except (KeyError, TypeError) as e:
        raise ValueError(f"{path}: not a dump_pruned_model pickle ({e})") from None
    layers = []
    for mname, mval in masks.items():
        scope = mname.rsplit("/", 1)[0] if "/" in mname else ""
        kname = next((k for k in masked if k.rsplit("/", 1)[0] == scope and "kernel" in k.rsplit("/", 1)[-1]), None)
        if kname is None:
            raise ValueError(f"{mname}: no masked kernel in the same scope")
        mask = np.asarray(mval) != 0
        mk = np.asarray(masked[kname])
        if mask.shape != mk.shape:
            raise ValueError(f"{mname}: mask {mask.shape} and kernel {mk.shape} differ in shape")
        bname = next((k for k in origin if k.rsplit("/", 1)[0] == scope and "bias" in k.rsplit("/", 1)[-1]), None)
        layers.append({"name": kname, "kernel": np.asarray(origin.get(kname, mk)), "masked_kernel": mk,
                       "mask": mask, "bias": None if bname is None else np.asarray(origin[bname])})
    return layers


def tiles_from_dumped_layer(layer: dict, G: int = 128, strict: bool = False):
    """One layer of `load_bert_dumped_model` as (TileSet, residual): its `absolute_mask` read like any
    other reference mask (`tiles_from_reference_mask`); pack `layer["masked_kernel"]` or `layer["kernel"]`."""
    return tiles_from_reference_mask(layer["mask"], G, strict)
