"""Seeded synthetic inputs with the shapes and value distributions of the benchmark configurations.

The reference measured on ImageNet / GLUE / IWSLT15 models and on unseeded rand() matrices
(StreamMaskedGEMM/perf/basic_nn.cu:612-620); none of those inputs exist here, so seeded NumPy
generators with the same shapes and distributions stand in.
"""
from __future__ import annotations

import numpy as np

# name -> (K, N): the GEMMs of one BERT-base encoder layer (hidden 768, FFN 3072).
BERT_BASE_LAYER = {"qkv": (768, 2304), "attn_out": (768, 768), "ffn1": (768, 3072), "ffn2": (3072, 768)}
BERT_SEEDS = {"qkv": 2001, "attn_out": 2002, "ffn1": 2003, "ffn2": 2004}


def rng(seed: int) -> np.random.Generator:
    return np.random.Generator(np.random.PCG64(seed))


def bert_gemm(name: str, M: int = 4096):
    """(A[M, K] ~ N(0,1), W[K, N] ~ N(0, 0.02)) as float32."""
    K, N = BERT_BASE_LAYER[name]
    g = rng(BERT_SEEDS[name])
    A = g.standard_normal((M, K), dtype=np.float32)
    W = (g.standard_normal((K, N), dtype=np.float32) * np.float32(0.02)).astype(np.float32)
    return A, W


def random_kept_lists(K: int, n_tiles: int, keep: int, seed: int):
    """Per-tile sorted random subsets of `keep` rows out of K, the perf driver's synthetic masks
    (mask_gen, basic_nn.cu:697-718) with a seed."""
    g = rng(seed)
    return [np.sort(g.permutation(K)[:keep]).astype(np.int32) for _ in range(n_tiles)]


def beta_skewed_counts(K: int, n_tiles: int, keep_frac: float, seed: int) -> np.ndarray:
    """Per-tile kept-row counts with keep fractions ~ Beta(2,5), rescaled to sum to
    keep_frac*K*n_tiles, rounded to multiples of 8 and clipped to [8, K]."""
    g = rng(seed)
    f = g.beta(2.0, 5.0, size=n_tiles)
    f = f * (keep_frac * n_tiles / f.sum())
    return np.clip(np.round(f * K / 8).astype(np.int64) * 8, 8, K).astype(np.int32)
