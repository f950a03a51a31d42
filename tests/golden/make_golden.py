"""Generates tests/golden/tw_masks.npz by running the REFERENCE's mask builder, unmodified.

Run in a container that has the reference checkout (default /root/reference):

    python tests/golden/make_golden.py [path-to-reference]

It imports Pruning/VGG/prune_algo.py from the reference tree and calls
pruning_fun(name)(scores, sparsity[, granularity][, g1percent]) (prune_algo.py:267-278) on seeded
inputs; the resulting 0/1 masks are stored bit-packed.  Inputs are not stored: `case_inputs`
regenerates them from the seed, and the tests call it too.  Seeded synthetic weights stand in for
the trained networks the reference pruned (N(0, 0.02) like BERT's initialiser, He-normal for the
conv kernel, U(-0.1, 0.1) like the NMT LSTM).
"""
from __future__ import annotations

import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))

# name -> (algorithm, list of layer shapes, sparsity, granularity, g1percent or None, seed, dist)
CASES = {
    "tw1_small":        ("tw1", [(96, 320)], 75.0, 128, None, 11, "normal"),
    "tw1_group":        ("tw1", [(64, 256), (80, 200), (48, 130)], 60.0, 128, None, 12, "normal"),
    "tw1_g32":          ("tw1", [(128, 160)], 50.0, 32, None, 13, "uniform"),
    "tw1_bert_ffn1":    ("tw1", [(768, 3072)], 75.0, 128, None, 2003, "bert"),
    "tw1_narrow":       ("tw1", [(40, 100)], 90.0, 128, None, 14, "normal"),
    "tw2_small":        ("tw2", [(96, 384)], 75.0, 128, None, 21, "normal"),
    "tw2_group":        ("tw2", [(64, 300), (72, 260)], 50.0, 64, None, 22, "normal"),
    "tw2_conv":         ("tw2", [(3, 3, 32, 160)], 75.0, 64, None, 23, "he"),
    "tw1m_small":       ("tw1m", [(96, 320)], 70.0, 128, 5.0, 31, "normal"),
    "tw1m_lstm":        ("tw1m", [(256, 512), (128, 512)], 75.0, 128, 1.5, 32, "uniform"),
    "tw2m_small":       ("tw2m", [(96, 384)], 70.0, 128, 1.0, 41, "normal"),
    # baseline patterns (no granularity argument): element-wise and vector-wise
    "ew_small":         ("ew", [(96, 320)], 75.0, None, None, 51, "normal"),
    "ew_group":         ("ew", [(64, 256), (80, 200), (48, 130)], 62.5, None, None, 52, "normal"),
    "ew_bert_attn":     ("ew", [(768, 768)], 90.0, None, None, 2002, "bert"),
    "vw_small":         ("vw", [(96, 320)], 75.0, None, None, 61, "normal"),
    "vw_ragged":        ("vw", [(70, 130), (16, 40), (9, 33)], 50.0, None, None, 62, "uniform"),
    "vw_90":            ("vw", [(128, 96)], 90.0, None, None, 63, "normal"),
}


def case_inputs(name: str):
    """The seeded score matrices of a case, as the reference's hooks hand them over: 2-D arrays of
    absolute values (img2col_forward, prune_algo.py:16-24, reshapes HWIO kernels and takes abs)."""
    algo, shapes, sparsity, gran, g1, seed, dist = CASES[name]
    g = np.random.Generator(np.random.PCG64(seed))
    out = []
    for shp in shapes:
        if dist == "uniform":
            w = g.uniform(-0.1, 0.1, size=shp).astype(np.float32)
        elif dist == "he":
            w = (g.standard_normal(shp, dtype=np.float32) * np.float32(np.sqrt(2.0 / np.prod(shp[:-1]))))
        elif dist == "bert":
            g.standard_normal((4096, shp[0]), dtype=np.float32)   # same stream position as synth.bert_gemm
            w = g.standard_normal(shp, dtype=np.float32) * np.float32(0.02)
        else:
            w = g.standard_normal(shp, dtype=np.float32) * np.float32(0.02)
        w = w.astype(np.float32)
        if w.ndim == 4:
            w = w.reshape(-1, w.shape[3])
        out.append(np.abs(w))
    return out


def main():
    ref = sys.argv[1] if len(sys.argv) > 1 else "/root/reference"
    sys.path.insert(0, os.path.join(ref, "Pruning", "VGG"))
    import prune_algo  # the reference's own module
    store = {}
    for name, (algo, shapes, sparsity, gran, g1, seed, dist) in CASES.items():
        scores = case_inputs(name)
        fn = prune_algo.pruning_fun(algo)
        if gran is None:
            masks = fn(scores, sparsity)
        else:
            masks = fn(scores, sparsity, gran) if g1 is None else fn(scores, sparsity, gran, g1)
        for i, m in enumerate(masks):
            m = np.asarray(m).astype(bool)
            store[f"{name}/{i}/shape"] = np.asarray(m.shape, dtype=np.int32)
            store[f"{name}/{i}/bits"] = np.packbits(m.reshape(-1))
        print(name, [float(np.asarray(m).mean()) for m in masks])
    np.savez_compressed(os.path.join(HERE, "tw_masks.npz"), **store)


def load_golden(name: str):
    """The reference's masks of a case, as a list of bool arrays."""
    z = np.load(os.path.join(HERE, "tw_masks.npz"))
    out, i = [], 0
    while f"{name}/{i}/shape" in z:
        shp = tuple(int(v) for v in z[f"{name}/{i}/shape"])
        out.append(np.unpackbits(z[f"{name}/{i}/bits"])[:shp[0] * shp[1]].reshape(shp).astype(bool))
        i += 1
    return out


if __name__ == "__main__":
    main()
