"""Seeded synthetic workloads with the shapes, sizes and value distributions of the five
benchmark configurations.  They stand in for the graph datasets the reference trains on
(OGB products / papers100M / MAG240M), which are not available offline.

Everything is generated with numpy's PCG64 (``seed = 1000 * config + rank``) so that the
same arrays come out on every machine.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np


def rng_for(config: int, rank: int = 0, stream: int = 0) -> np.random.Generator:
    return np.random.default_rng([1000 * config + rank, stream])


def rank_to_id(ranks: np.ndarray, num_ids: int, salt: int = 0x9E3779B97F4A7C15) -> np.ndarray:
    """A fixed pseudo-random permutation of [0, num_ids): popularity rank -> node id, so
    that hot ids are scattered over the id space (otherwise ``id % lines`` never
    collides).  Invertible mixing on the next power of two, cycle-walked into range."""
    ranks = np.asarray(ranks, dtype=np.uint64)
    k = max(int(num_ids - 1).bit_length(), 2)
    mask = np.uint64((1 << k) - 1)
    m1 = np.uint64((salt | 1) & ((1 << 64) - 1))
    m2 = np.uint64(0xD6E8FEB86659FD93)
    s1 = np.uint64(max(k // 2, 1))
    s2 = np.uint64(max(k // 3, 1))

    def mix(x):
        x = (x * m1) & mask
        x ^= x >> s1
        x = (x * m2) & mask
        x ^= x >> s2
        x = (x * m1) & mask
        x ^= x >> s1
        return x

    with np.errstate(over="ignore"):
        out = mix(ranks)
        bad = out >= np.uint64(num_ids)
        while bad.any():
            out[bad] = mix(out[bad])
            bad = out >= np.uint64(num_ids)
    return out.astype(np.int64)


class ZipfSampler:
    """Bounded Zipf(s) over ranks [0, num_ids) by inverse CDF (exact discrete CDF)."""

    def __init__(self, num_ids: int, s: float):
        w = np.arange(1, num_ids + 1, dtype=np.float64) ** (-s)
        self.cdf = np.cumsum(w)
        self.cdf /= self.cdf[-1]
        self.num_ids = num_ids

    def ranks(self, rng: np.random.Generator, n: int) -> np.ndarray:
        u = rng.random(n)
        return np.minimum(np.searchsorted(self.cdf, u, side="left"), self.num_ids - 1).astype(np.int64)

    def ids(self, rng: np.random.Generator, n: int) -> np.ndarray:
        return rank_to_id(self.ranks(rng, n), self.num_ids)

    def unique_ranks(self, rng: np.random.Generator, n: int) -> np.ndarray:
        """n distinct popularity ranks, Zipf-weighted without replacement (draw, de-duplicate
        in draw order, top up)."""
        have = np.empty(0, dtype=np.int64)
        while have.size < n:
            draw = self.ranks(rng, int((n - have.size) * 1.5) + 16)
            cat = np.concatenate([have, draw])
            _, first = np.unique(cat, return_index=True)
            have = cat[np.sort(first)]
        return have[:n]

    def unique_ids(self, rng: np.random.Generator, n: int, id_space: int | None = None) -> np.ndarray:
        """n distinct ids; id_space: spread the ranks over a larger id space than the ranking
        (a ranking truncated to its head keeps the CDF small for very large tables)."""
        return rank_to_id(self.unique_ranks(rng, n), self.num_ids if id_space is None else id_space)


def hot_ids(num_ids: int, count: int) -> np.ndarray:
    """The ids of the `count` most popular ranks, in rank order."""
    return rank_to_id(np.arange(count, dtype=np.int64), num_ids)


def normal_rows(rng: np.random.Generator, n: int, dim: int, sigma: float) -> np.ndarray:
    return (rng.standard_normal((n, dim), dtype=np.float32) * np.float32(sigma)).astype(np.float32)


@dataclass(frozen=True)
class CacheFetchConfig:
    """Cached fetch / set workloads (configurations 1 and 2)."""
    name: str
    config: int
    table_rows: int
    dim: int
    cache_entries: int
    batch: int
    zipf_s: float
    table_sigma: float = 0.01
    grad_sigma: float = 1e-3
    flush_every: int = 8


CONFIG1 = CacheFetchConfig("c1_cpu_runnable", 1, 1_000_000, 128, 100_000, 65_536, 1.1)
CONFIG2 = CacheFetchConfig("c2_single_b200", 2, 20_000_000, 128, 4_000_000, 2_000_000, 1.2)


def scaled(cfg: CacheFetchConfig, factor: float, name: str | None = None) -> CacheFetchConfig:
    """The same workload with every size multiplied by `factor` (tests, ncu captures)."""
    return CacheFetchConfig(name or f"{cfg.name}_x{factor:g}", cfg.config,
                            max(int(cfg.table_rows * factor), 1024), cfg.dim,
                            max(int(cfg.cache_entries * factor), 64),
                            max(int(cfg.batch * factor), 32), cfg.zipf_s, cfg.table_sigma,
                            cfg.grad_sigma, cfg.flush_every)


def stream_stats(ids: np.ndarray) -> dict:
    """Reported properties of an id stream (duplicate fraction is an output, not an
    assumption)."""
    u = np.unique(ids).size
    return {"n": int(ids.size), "unique": int(u), "duplicate_fraction": float(1.0 - u / max(ids.size, 1))}


# ---------------------------------------------------------------------------------------
# configuration 5: sampled 2-layer GraphSAGE frontier on a synthetic R-MAT graph
# ---------------------------------------------------------------------------------------
@dataclass(frozen=True)
class RmatConfig:
    """R-MAT(a, b, c, d) over 2**bits >= num_nodes vertices; the edge list is never
    materialised: a neighbour of u is drawn bit by bit from the conditional quadrant
    probabilities given u's bits (source bit 0: P(dest bit 0) = a/(a+b); source bit 1:
    c/(c+d)), redrawn while it falls outside [0, num_nodes)."""
    name: str = "c5_graphsage_rmat"
    config: int = 5
    num_nodes: int = 100_000_000
    bits: int = 27
    a: float = 0.57
    b: float = 0.19
    c: float = 0.19
    seeds: int = 1024
    fanout: tuple = (25, 10)
    dim: int = 128
    cache_entries: int = 4_000_000
    hot_popcount: int = 7       # ids with at most this many one-bits are "hot" (about 1 % of the ids)
    table_sigma: float = 0.01
    grad_sigma: float = 1e-3
    flush_every: int = 8

    @property
    def table_rows(self) -> int:
        return self.num_nodes

    @property
    def batch(self) -> int:
        n, total = self.seeds, self.seeds
        for f in self.fanout:
            n *= f
            total += n
        return total


CONFIG5 = RmatConfig()


def scaled_rmat(cfg: RmatConfig, bits: int, seeds: int | None = None, name: str | None = None) -> RmatConfig:
    """The same sampler on a smaller graph (tests, captures): 2**bits vertices, 3/4 of them used."""
    return RmatConfig(name or f"{cfg.name}_b{bits}", cfg.config, (3 << bits) // 4, bits, cfg.a, cfg.b, cfg.c,
                      seeds or cfg.seeds, cfg.fanout, cfg.dim, max((3 << bits) // 100, 64),
                      max(bits // 4, 1), cfg.table_sigma, cfg.grad_sigma, cfg.flush_every)


def rmat_neighbors(cfg: RmatConfig, src: np.ndarray, fanout: int, rng: np.random.Generator) -> np.ndarray:
    """fanout sampled neighbours of every vertex in src, shape [len(src) * fanout]."""
    u = np.repeat(np.asarray(src, dtype=np.int64), fanout)
    d = 1.0 - cfg.a - cfg.b - cfg.c
    p0_s0 = cfg.a / (cfg.a + cfg.b)
    p0_s1 = cfg.c / (cfg.c + d)
    out = np.empty_like(u)
    todo = np.arange(u.size)
    while todo.size:
        v = np.zeros(todo.size, dtype=np.int64)
        uu = u[todo]
        for level in range(cfg.bits - 1, -1, -1):
            sbit = (uu >> level) & 1
            p0 = np.where(sbit == 0, p0_s0, p0_s1)
            v |= (rng.random(todo.size) >= p0).astype(np.int64) << level
        ok = v < cfg.num_nodes
        out[todo[ok]] = v[ok]
        todo = todo[~ok]
    return out


def rmat_frontier(cfg: RmatConfig, rng: np.random.Generator) -> np.ndarray:
    """All vertices whose embeddings one step fetches: the seeds and their sampled 1-hop and
    2-hop neighbours, duplicates kept (the embedding layer de-duplicates gradients, not ids)."""
    layer = rng.integers(0, cfg.num_nodes, cfg.seeds, dtype=np.int64)
    parts = [layer]
    for f in cfg.fanout:
        layer = rmat_neighbors(cfg, layer, f, rng)
        parts.append(layer)
    return np.concatenate(parts)
