"""Seeded synthetic inputs with the reference's shapes and value distributions (host side, numpy).

The reference trains on Tiny Shakespeare bytes, which cannot be fetched here; the stand-in is a corpus of
bytes drawn i.i.d. from Zipf(s = 1.1) over 256 symbols, sampled into [B][T+1] windows the way the
reference's ByteDataset::sample_batch_packed does (src/dataset.cpp:39-54). Weight initialisation follows
the reference's seeds (src/train_efla_lm.cpp:4889-4921, TernaryMatrix::init_rand :174-183).
"""
from __future__ import annotations

import numpy as np

_GOLD = np.uint64(0x9E3779B97F4A7C15)


def splitmix64_stream(seed: int, n: int) -> np.ndarray:
    """The first n outputs of splitmix64 started at `seed` (reference: src/rng.h:7-12), vectorised."""
    with np.errstate(over="ignore"):
        i = np.arange(1, n + 1, dtype=np.uint64)
        z = np.uint64(seed) + i * _GOLD
        z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        return z ^ (z >> np.uint64(31))


def mix(a: int, b: int) -> int:
    """The reference's seed mixer (src/rng.h:14-29): seeds of an epoch's batch, of a pair, of a matrix."""
    m = (1 << 64) - 1
    a &= m
    b &= m
    x = a ^ ((b + 0x9E3779B97F4A7C15 + (a << 6) + (a >> 2)) & m)
    x ^= x >> 33
    x = (x * 0xFF51AFD7ED558CCD) & m
    x ^= x >> 33
    x = (x * 0xC4CEB9FE1A85EC53) & m
    x ^= x >> 33
    return x


def ternary_from_u64(x: np.ndarray) -> np.ndarray:
    r = (x & np.uint64(0xFF)).astype(np.int32)
    return np.where(r < 85, -1, np.where(r < 170, 0, 1)).astype(np.int8)


def init_rand_ternary(shape, seed: int) -> np.ndarray:
    n = int(np.prod(shape))
    return ternary_from_u64(splitmix64_stream(seed, n)).reshape(shape)


def init_weights(cfg) -> dict:
    """cfg: bitnet_nvfp4_b200.population.Config"""
    V, H, L, F, T = cfg.vocab, cfg.hidden, cfg.layers, cfg.hidden * cfg.mlp_mult, cfg.seq
    w = {
        "emb": init_rand_ternary((V, H), 0x1000),
        "win": init_rand_ternary((H, H), 0x2000),
        "wq": np.stack([init_rand_ternary((H, H), 0x3000 + 8 * l + 0) for l in range(L)]),
        "wk": np.stack([init_rand_ternary((H, H), 0x3000 + 8 * l + 1) for l in range(L)]),
        "wv": np.stack([init_rand_ternary((H, H), 0x3000 + 8 * l + 2) for l in range(L)]),
        "wbeta": np.stack([init_rand_ternary((H,), 0x3000 + 8 * l + 3) for l in range(L)]),
        "ff1": np.stack([init_rand_ternary((F, H), 0x3000 + 8 * l + 4) for l in range(L)]),
        "ff2": np.stack([init_rand_ternary((H, F), 0x3000 + 8 * l + 5) for l in range(L)]),
        "head": init_rand_ternary((V, H), 0x7000),
        "head_bias": np.zeros(V, np.float32),
        "beta_bias": np.full(L, -2.0, np.float32),
    }
    u = (splitmix64_stream(0xABCDEF, T * H) & np.uint64(0xFFFF)).astype(np.float32) / np.float32(65535.0)
    w["pos"] = ((u - np.float32(0.5)) * np.float32(0.04)).astype(np.float32).reshape(T, H)
    return w


def zipf_corpus(n_bytes: int = 1 << 20, s: float = 1.1, seed: int = 123) -> np.ndarray:
    """n_bytes symbols with P(rank r) ~ r^-s over 256 symbols, by inverse-CDF sampling of splitmix64 outputs."""
    ranks = np.arange(1, 257, dtype=np.float64)
    p = ranks ** (-s)
    cdf = np.cumsum(p / p.sum())
    u = (splitmix64_stream(seed, n_bytes) >> np.uint64(11)).astype(np.float64) * (1.0 / (1 << 53))
    return np.minimum(np.searchsorted(cdf, u, side="right"), 255).astype(np.uint8)


def load_corpus(path) -> np.ndarray:
    """A real byte corpus (e.g. Tiny Shakespeare) as the reference's ByteDataset::load_file reads it (src/dataset.cpp:8-20)."""
    data = np.fromfile(path, dtype=np.uint8)
    if data.size < 2:
        raise ValueError("dataset too small")
    return data


def sample_batch(corpus: np.ndarray, batch: int, seq: int, seed: int):
    """(tokens, targets) uint8 [batch][seq]: window starts from splitmix64(seed) % (len - seq - 1)."""
    r = splitmix64_stream(seed, batch)
    starts = (r % np.uint64(len(corpus) - seq - 1)).astype(np.int64)
    idx = starts[:, None] + np.arange(seq + 1)[None, :]
    win = corpus[idx]
    return np.ascontiguousarray(win[:, :seq]), np.ascontiguousarray(win[:, 1:])
