"""Generates tests/golden/tw_masks.npz by running the REFERENCE's mask builder, unmodified.

Run where a checkout of the reference repository is available:

    python tests/golden/make_golden.py <path-to-reference-checkout>

It imports Pruning/VGG/prune_algo.py from the reference tree and calls
pruning_fun(name)(scores, sparsity[, granularity][, g1percent]) (prune_algo.py:267-278) on seeded
inputs; the resulting 0/1 masks are stored bit-packed.  The BERT variants live in
Pruning/BERT/utils/MyHook.py, whose only TensorFlow uses at import time are the module-level import
and two `tf.train.SessionRunHook` base classes; a stub module with that one attribute lets the file be
imported as it is, and `granularity_pruning` (:202-214, pruning type 2) and `pruning(...)` types 7 and
8 (:216-313) are then called directly, with a stand-in session that captures the masks the function
feeds to its assign ops.  Inputs are not stored: `case_inputs` regenerates them from the seed, and
the tests call it too.  Seeded synthetic weights stand in for the trained networks the reference
pruned (N(0, 0.02) like BERT's initialiser, He-normal for the conv kernel, U(-0.1, 0.1) like the NMT
LSTM).
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
    # benchmark-configuration sizes: VGG16 conv5 as a 4608 x 512 matrix, the NMT LSTM gate matrix
    "tw2_vgg_conv5":    ("tw2", [(3, 3, 512, 512)], 75.0, 128, None, 3001, "he"),
    "tw1m_nmt_lstm":    ("tw1m", [(2048, 4096)], 75.0, 128, 1.5, 4001, "uniform"),
    # Taylor scores: float64 arrays, three steps of square(grad * w) in float32 accumulated in double
    # (what the reference's hooks hand to pruning_fun after score accumulation, myhook.py:248-257)
    "tw1_taylor64":     ("tw1", [(96, 320)], 75.0, 128, None, 81, "taylor"),
    "tw1_taylor64_grp": ("tw1", [(3, 3, 16, 96), (200, 333)], 62.5, 64, None, 82, "taylor"),
    "tw1_taylor64_ffn": ("tw1", [(768, 3072)], 75.0, 128, None, 83, "taylor"),
    # baseline patterns (no granularity argument): element-wise and vector-wise
    "ew_small":         ("ew", [(96, 320)], 75.0, None, None, 51, "normal"),
    "ew_group":         ("ew", [(64, 256), (80, 200), (48, 130)], 62.5, None, None, 52, "normal"),
    "ew_bert_attn":     ("ew", [(768, 768)], 90.0, None, None, 2002, "bert"),
    "vw_small":         ("vw", [(96, 320)], 75.0, None, None, 61, "normal"),
    "vw_ragged":        ("vw", [(70, 130), (16, 40), (9, 33)], 50.0, None, None, 62, "uniform"),
    "vw_90":            ("vw", [(128, 96)], 90.0, None, None, 63, "normal"),
    # block-wise (32 x 32 blocks, the default its hooks use); norms via the generating host's BLAS
    "bw_small":         ("bw", [(96, 320)], 75.0, None, None, 91, "normal"),
    "bw_ragged":        ("bw", [(70, 130), (40, 33)], 50.0, None, None, 92, "uniform"),
    "bw_bert_attn":     ("bw", [(768, 768)], 90.0, None, None, 2002, "bert"),
}


# BERT pruning types (Pruning/BERT/utils/MyHook.py): name -> (type, shapes, sparsity, granularity, seed, dist).
# Type 2 prunes one matrix at a time; types 7 and 8 take the whole list under one threshold and need
# 768 % granularity == 0 and N % granularity == 0.
BERT_CASES = {
    "bert2_small":      (2, [(96, 256)], 75.0, 128, 71, "normal"),
    "bert2_ffn1":       (2, [(768, 3072)], 75.0, 128, 2003, "bert"),
    "bert2_g64":        (2, [(128, 384)], 40.0, 64, 72, "uniform"),
    "bert7_group":      (7, [(96, 256), (64, 384)], 60.0, 128, 73, "normal"),
    "bert7_attn":       (7, [(768, 768)], 75.0, 128, 2002, "bert"),
    "bert8_group":      (8, [(96, 384), (72, 256)], 50.0, 64, 74, "normal"),
    "bert8_qkv":        (8, [(768, 2304)], 50.0, 128, 2001, "bert"),
}


def taylor_steps(g, shp, steps: int = 3):
    """(weights, accumulated scores): per step square(grad * w) in float32 (compute_taylor_score,
    Pruning/VGG/myhook.py:44-48) added into a float64 array (after_run, :248-257)."""
    w = (g.standard_normal(shp, dtype=np.float32) * np.float32(0.05)).astype(np.float32)
    acc = np.zeros(shp)
    grads = []
    for _ in range(steps):
        grad = g.standard_normal(shp, dtype=np.float32)
        grads.append(grad)
        t = (grad * w).astype(np.float32)
        acc += (t * t).astype(np.float32)
    return (w, grads), acc


def case_inputs(name: str):
    """The seeded score matrices of a case, as the reference's hooks hand them over: 2-D arrays of
    absolute values (img2col_forward, prune_algo.py:16-24, reshapes HWIO kernels and takes abs)."""
    if name in BERT_CASES:
        _, shapes, sparsity, gran, seed, dist = BERT_CASES[name]
    else:
        algo, shapes, sparsity, gran, g1, seed, dist = CASES[name]
    g = np.random.Generator(np.random.PCG64(seed))
    out = []
    for shp in shapes:
        if dist == "taylor":
            w, acc = taylor_steps(g, shp)
            if acc.ndim == 4:
                acc = acc.reshape(-1, acc.shape[3])
            out.append(np.abs(acc))
            continue
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


def import_bert_hook(ref: str):
    """The reference's Pruning/BERT/utils/MyHook.py, imported unmodified next to a stub `tensorflow`
    module that provides the one attribute the file touches while it is being imported."""
    import importlib.util
    import types
    if "tensorflow" not in sys.modules:
        tf = types.ModuleType("tensorflow")
        tf.train = types.SimpleNamespace(SessionRunHook=object)
        sys.modules["tensorflow"] = tf
    spec = importlib.util.spec_from_file_location(
        "reference_bert_myhook", os.path.join(ref, "Pruning", "BERT", "utils", "MyHook.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


class _Placeholder:
    """Stands in for a TF placeholder: hashable, with the shape the reference asserts on."""

    def __init__(self, shape):
        self.shape = tuple(shape)


class _Session:
    """Stands in for tf.Session: keeps the feed dict of the one `run(assign_ops, feed)` call."""

    def __init__(self):
        self.feed = None

    def run(self, ops, feed):
        self.feed = feed


def run_bert_case(hook_mod, name: str):
    ptype, shapes, sparsity, gran, seed, dist = BERT_CASES[name]
    scores = case_inputs(name)
    pruner = hook_mod.SparseColumnPruningRank()
    if ptype == 2:
        return [pruner.granularity_pruning(768, gran, sc, sparsity) for sc in scores]
    ph = [_Placeholder(sc.shape) for sc in scores]
    sess = _Session()
    pruner.pruning("golden", scores, sparsity, ph, sess, None, ptype, gran)
    return [sess.feed[p] for p in ph]


def main():
    if len(sys.argv) < 2:
        raise SystemExit("usage: make_golden.py <path-to-reference-checkout>")
    ref = sys.argv[1]
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
    hook_mod = import_bert_hook(ref)
    for name in BERT_CASES:
        masks = run_bert_case(hook_mod, name)
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
