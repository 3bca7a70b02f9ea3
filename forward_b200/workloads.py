"""Seeded synthetic EmbeddingBag workloads (numpy, host side).

These stand in for recommender-style lookups: only shapes, bag-length laws and
index distributions are modelled; no public dataset is read or reproduced.
Draw order inside each generator is fixed (lengths, then indices, then extras)
so a seed names one input exactly.

Index laws
----------
``uniform``  every row equally likely.
``zipf``     rank r (1-based) has probability proportional to r**-s over the
             finite set of rows (inverse-CDF on the normalised pmf); ranks are
             mapped to rows through a seeded permutation so hot rows are spread
             over the table rather than packed at its start.
"""
from __future__ import annotations

import dataclasses

import numpy as np


@dataclasses.dataclass
class Bags:
    """One batch of lookups in the 1-D indices + offsets form (or fixed length)."""
    indices: np.ndarray              # int32 [N]
    offsets: np.ndarray | None       # int32 [B]; None when fixed_len > 0
    fixed_len: int = 0
    per_sample_weights: np.ndarray | None = None  # fp32 [N]

    @property
    def num_bags(self) -> int:
        return self.indices.size // self.fixed_len if self.fixed_len else self.offsets.size

    @property
    def num_indices(self) -> int:
        return int(self.indices.size)


def offsets_from_lengths(lengths: np.ndarray) -> np.ndarray:
    off = np.zeros(lengths.size, dtype=np.int64)
    np.cumsum(lengths[:-1], out=off[1:])
    return off


class ZipfSampler:
    """Inverse-CDF sampler of a finite Zipf law with a seeded rank->row permutation."""

    def __init__(self, num_rows: int, s: float, rng: np.random.Generator, permute: bool = True):
        ranks = np.arange(1, num_rows + 1, dtype=np.float64)
        pmf = ranks ** (-s)
        self.cdf = np.cumsum(pmf)
        self.cdf /= self.cdf[-1]
        self.perm = rng.permutation(num_rows).astype(np.int64) if permute else None
        self.num_rows = num_rows

    def draw(self, n: int, rng: np.random.Generator) -> np.ndarray:
        u = rng.random(n)
        rank0 = np.searchsorted(self.cdf, u, side="left")
        np.minimum(rank0, self.num_rows - 1, out=rank0)
        return self.perm[rank0] if self.perm is not None else rank0


def ragged_bags(num_rows: int, lengths: np.ndarray, rng: np.random.Generator, *,
                law: str = "uniform", zipf_s: float = 1.05,
                sampler: ZipfSampler | None = None) -> Bags:
    n = int(lengths.sum())
    if law == "uniform":
        idx = rng.integers(0, num_rows, n, dtype=np.int64)
    elif law == "zipf":
        sampler = sampler or ZipfSampler(num_rows, zipf_s, rng)
        idx = sampler.draw(n, rng)
    else:
        raise ValueError(law)
    return Bags(idx.astype(np.int32), offsets_from_lengths(lengths).astype(np.int32))


# ---- the five named configurations ---------------------------------------------

def config1(seed: int = 0):
    """10 000 x 64 fp32 N(0,1), 32 bags of 1..20 uniform indices, sum."""
    rng = np.random.default_rng(seed)
    table = rng.standard_normal((10_000, 64), dtype=np.float32)
    lengths = rng.integers(1, 21, 32)
    return table, ragged_bags(10_000, lengths, rng)


def config2_bags(seed: int = 1, *, num_rows: int = 1_000_000, num_bags: int = 16384,
                 sampler: ZipfSampler | None = None,
                 rng: np.random.Generator | None = None) -> Bags:
    """Bag lengths Poisson(40) clipped to [1, 200]; indices Zipf(1.05) over the rows."""
    rng = rng or np.random.default_rng(seed)
    lengths = np.clip(rng.poisson(40.0, num_bags), 1, 200)
    return ragged_bags(num_rows, lengths, rng, law="zipf", zipf_s=1.05, sampler=sampler)


def config2_table(seed: int = 1, num_rows: int = 1_000_000, dim: int = 128) -> np.ndarray:
    """fp16 table, N(0, 0.1) rounded to half."""
    rng = np.random.default_rng(seed + 1000)
    return (rng.standard_normal((num_rows, dim), dtype=np.float32) * 0.1).astype(np.float16)


def config3_bags(seed: int = 2, *, num_rows: int = 4_000_000, num_bags: int = 8192) -> Bags:
    """Lengths uniform 0..64 (empty bags included), uniform indices, 5 % set to 0 (= padding)."""
    rng = np.random.default_rng(seed)
    lengths = rng.integers(0, 65, num_bags)
    bags = ragged_bags(num_rows, lengths, rng)
    hit = rng.random(bags.indices.size) < 0.05
    bags.indices[hit] = 0
    return bags


def config4_rows(seed: int = 3, num_tables: int = 26) -> np.ndarray:
    """Row counts log-uniform in [1e3, 4e7]."""
    rng = np.random.default_rng(seed)
    return np.round(np.exp(rng.uniform(np.log(1e3), np.log(4e7), num_tables))).astype(np.int64)


def config4_bags(table_id: int, num_rows: int, seed: int = 3, *, batch: int = 65536,
                 pooling: int = 20) -> Bags:
    """Fixed pooling factor, Zipf(1.1) indices, per-sample weights U(0,1)."""
    rng = np.random.default_rng([seed, table_id])
    sampler = ZipfSampler(num_rows, 1.1, rng)
    idx = sampler.draw(batch * pooling, rng).astype(np.int32)
    w = rng.random(batch * pooling, dtype=np.float32)
    return Bags(idx, None, fixed_len=pooling, per_sample_weights=w)


def config5_bags(seed: int = 4, *, num_rows: int = 1_000_000_000, num_bags: int = 131072) -> Bags:
    """Lengths uniform 1..100, uniform indices over the whole (sharded) table."""
    rng = np.random.default_rng(seed)
    lengths = rng.integers(1, 101, num_bags)
    return ragged_bags(num_rows, lengths, rng)


def algorithmic_bytes(*, gathered_rows: int, dim: int, table_itemsize: int, num_indices: int,
                      num_offsets: int, index_itemsize: int, num_bags: int, out_itemsize: int,
                      weighted: bool = False) -> int:
    """Bytes one call must move: rows read + indices + offsets (+ weights) + output.

    Repeated rows are counted every time and cache hits earn no credit."""
    return (gathered_rows * dim * table_itemsize + num_indices * index_itemsize
            + num_offsets * index_itemsize + (num_indices * 4 if weighted else 0)
            + num_bags * dim * out_itemsize)
