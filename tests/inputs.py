"""Seeded synthetic inputs with the shapes and value distributions of the
benchmark configurations (no dataset is involved anywhere)."""
from __future__ import annotations

import numpy as np

N_EMBD, HEAD_DIM, N_ROT, FF_DIM, TOP_K, VOCAB, N_HC = 4096, 512, 64, 2048, 6, 129280, 4
EPS, CLAMP, SINKHORN_ITERS = 1e-6, 10.0, 20


def rng(seed: int) -> np.random.Generator:
    return np.random.default_rng(seed)


def normal(g, shape, sigma=1.0):
    return (g.standard_normal(shape, dtype=np.float32) * np.float32(sigma)).astype(np.float32)


def uniform(g, shape, lo, hi):
    return g.uniform(lo, hi, shape).astype(np.float32)


def q8_0_table(g, vocab: int, n_embd: int) -> np.ndarray:
    """[vocab, n_embd/32, 34] uint8: f16 scale ~U(0.001,0.02) then 32 int8 ~U[-127,127]."""
    nb = n_embd // 32
    t = np.empty((vocab, nb, 34), dtype=np.uint8)
    d = g.uniform(0.001, 0.02, (vocab, nb)).astype(np.float16)
    t[:, :, 0:2] = d.view(np.uint8).reshape(vocab, nb, 2)
    t[:, :, 2:] = g.integers(-127, 128, (vocab, nb, 32), dtype=np.int8).view(np.uint8)
    return t


def f16_table(g, vocab: int, n_embd: int) -> np.ndarray:
    return (g.standard_normal((vocab, n_embd), dtype=np.float32) * 0.02).astype(np.float16)


def router_weights(g, T: int, k: int) -> np.ndarray:
    """softmax of N(0,1) logits over the k slots (the synthetic generator of the
    benchmark config; the hot path takes the weights as an input)."""
    z = g.standard_normal((T, k)).astype(np.float64)
    e = np.exp(z - z.max(axis=1, keepdims=True))
    return (e / e.sum(axis=1, keepdims=True)).astype(np.float32)


def config1(seed=1):
    """Single-token decode prologue."""
    g = rng(seed)
    return dict(
        x=normal(g, (1, N_EMBD)), w=uniform(g, (N_EMBD,), 0.5, 1.5),
        q=normal(g, (1, 64, HEAD_DIM)), pos=np.array([1234], dtype=np.int32),
        gate=normal(g, (1, 1, FF_DIM), 2.0), up=normal(g, (1, 1, FF_DIM), 2.0))


def config2(seed=2, T=4096, vocab=VOCAB, n_embd=N_EMBD):
    g = rng(seed)
    return dict(
        table=q8_0_table(g, vocab, n_embd), ids=g.integers(0, vocab, T).astype(np.int32),
        residual=normal(g, (T, n_embd)), w=uniform(g, (n_embd,), 0.5, 1.5))


def config3(seed=3, T=4096, head_dim=HEAD_DIM):
    g = rng(seed)
    return dict(kv=normal(g, (T, head_dim), 1.5), pos=np.arange(T, dtype=np.int32))


def config4(seed=4, T=4096, k=TOP_K, n=FF_DIM):
    g = rng(seed)
    return dict(gate=normal(g, (T, k, n), 2.0), up=normal(g, (T, k, n), 2.0),
                weights=router_weights(g, T, k))


def config5(seed=5, T=4096, n_embd=N_EMBD):
    g = rng(seed)
    return dict(resid=normal(g, (T, N_HC, n_embd)), logits=normal(g, (T, 16)))


def hc_pre_weights(seed=6, n_embd=N_EMBD):
    """hc_fn f16 [24, 4*n_embd] scaled so that mix is O(1); scale [3]; base [24]."""
    g = rng(seed)
    fn = (g.standard_normal((24, 4 * n_embd), dtype=np.float32) / np.sqrt(4 * n_embd)).astype(np.float16)
    return dict(fn=fn, scale=uniform(g, (3,), 0.5, 1.5), base=normal(g, (24,), 0.5))
