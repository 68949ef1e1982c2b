"""Seeded synthetic workloads with the shapes, sizes and value distributions of the five benchmark
configurations (single-row loop, Llama-3-vocab batch, large-vocab mixed batch, row-partitioned serving batch,
vocab-sharded batch).  They stand in for real LM-head logits; no dataset is used.

Everything is generated on the host with numpy's PCG64 so that the CPU checkers and the device see the same
bits.  Sampler seeds are never 0 (0 means "non-deterministic" in the reference, src/sampler.cpp:8).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import numpy as np

PARAMS_DTYPE = np.dtype(
    [
        ("temperature", "<f4"),
        ("top_k", "<i4"),
        ("top_p", "<f4"),
        ("min_p", "<f4"),
        ("repeat_penalty", "<f4"),
        ("repeat_last_n", "<i4"),
        ("seed", "<u8"),
    ]
)  # byte layout of qp::SamplerParams, include/qpack/engine.h:17-25


def make_params(n=1, temperature=0.7, top_k=40, top_p=0.9, min_p=0.05, repeat_penalty=1.1, repeat_last_n=64, seed=1):
    """n parameter blocks (structured array); each argument is a scalar or a length-n array.
    Defaults are the reference's (engine.h:18-24) except the seed."""
    p = np.zeros(n, dtype=PARAMS_DTYPE)
    p["temperature"] = temperature
    p["top_k"] = top_k
    p["top_p"] = top_p
    p["min_p"] = min_p
    p["repeat_penalty"] = repeat_penalty
    p["repeat_last_n"] = repeat_last_n
    p["seed"] = seed
    return p


@dataclass
class Workload:
    name: str
    logits: np.ndarray  # f32 [B, V]
    params: np.ndarray  # PARAMS_DTYPE [B] or [1]
    history: Optional[np.ndarray]  # i32 [B, H] or None
    hist_len: Optional[np.ndarray]  # i32 [B] or None

    @property
    def rows(self):
        return self.logits.shape[0]

    @property
    def vocab(self):
        return self.logits.shape[1]


def _normal(rng, shape, sigma):
    x = rng.standard_normal(shape, dtype=np.float32)
    x *= np.float32(sigma)
    return x


def _add_spikes(rng, logits, n_spikes, lo, hi, rows=None):
    B, V = logits.shape
    rows = np.arange(B) if rows is None else rows
    for r in rows:
        ids = rng.choice(V, size=n_spikes, replace=False)
        amt = rng.uniform(lo, hi, size=n_spikes).astype(np.float32) if hi > lo else np.full(n_spikes, lo, np.float32)
        logits[r, ids] += amt


def single_row_step(step: int, vocab: int = 151936, seed: int = 42) -> np.ndarray:
    """Config 1 logits for one step: f32 [1, vocab] ~ N(0, 2^2) with 16 spike ids raised by U(8, 14),
    regenerated from seed + step."""
    rng = np.random.Generator(np.random.PCG64(seed + step))
    x = _normal(rng, (1, vocab), 2.0)
    _add_spikes(rng, x, 16, 8.0, 14.0)
    return x


def single_row_loop(vocab: int = 151936, seed: int = 42):
    """Config 1: parameters and the initial 64-id history of the 1000-draw single-row loop."""
    rng = np.random.Generator(np.random.PCG64(seed ^ 0x5EED))
    params = make_params(1, temperature=0.8, top_k=40, top_p=0.95, min_p=0.05, repeat_penalty=1.1, repeat_last_n=64,
                         seed=seed)
    hist = rng.integers(0, vocab, size=64, dtype=np.int32)
    return params, hist


def llama3_batch(rows: int = 64, vocab: int = 128256, seed: int = 2) -> Workload:
    """Config 2: even rows flat N(0, 1), odd rows peaked N(0, 3^2) + 4 spikes at +12; temperature 1, top_p 0.9,
    top_k off, min_p off, no penalty; per-row seeds 1000 + row."""
    rng = np.random.Generator(np.random.PCG64(seed))
    x = _normal(rng, (rows, vocab), 1.0)
    odd = np.arange(1, rows, 2)
    x[odd] *= np.float32(3.0)
    _add_spikes(rng, x, 4, 12.0, 12.0, rows=odd)
    params = make_params(rows, temperature=1.0, top_k=0, top_p=0.9, min_p=0.0, repeat_penalty=1.0, repeat_last_n=64,
                         seed=1000 + np.arange(rows, dtype=np.uint64))
    return Workload("llama3_batch", x, params, None, None)


def mixed_batch(rows: int = 256, vocab: int = 201088, seed: int = 3, hist: int = 128) -> Workload:
    """Config 3: N(0, 2.5^2) + 8 spikes U(6, 15); heterogeneous per-row parameters: 25 % greedy, otherwise
    temperature U(0.5, 1.3), top_k in {0, 20, 50, 200}, top_p U(0.8, 1.0), min_p in {0, 0.05, 0.1};
    repeat_penalty U(1.0, 1.2) over 128 history ids per row; seeds 3000 + row."""
    rng = np.random.Generator(np.random.PCG64(seed))
    x = _normal(rng, (rows, vocab), 2.5)
    _add_spikes(rng, x, 8, 6.0, 15.0)
    greedy = rng.random(rows) < 0.25
    temp = rng.uniform(0.5, 1.3, rows).astype(np.float32)
    temp[greedy] = 0.0
    params = make_params(
        rows,
        temperature=temp,
        top_k=rng.choice(np.array([0, 20, 50, 200], np.int32), rows),
        top_p=rng.uniform(0.8, 1.0, rows).astype(np.float32),
        min_p=rng.choice(np.array([0.0, 0.05, 0.1], np.float32), rows),
        repeat_penalty=rng.uniform(1.0, 1.2, rows).astype(np.float32),
        repeat_last_n=hist,
        seed=3000 + np.arange(rows, dtype=np.uint64),
    )
    history = _history(rng, x, hist)
    return Workload("mixed_batch", x, params, history, np.full(rows, hist, np.int32))


def _history(rng, logits, n):
    """n history ids per row: mostly uniform over the vocabulary, a few taken from the row's top region so that
    the penalty actually moves candidates."""
    B, V = logits.shape
    h = rng.integers(0, V, size=(B, n), dtype=np.int32)
    n_top = max(1, n // 16)
    for r in range(B):
        top = np.argpartition(logits[r], V - 32)[V - 32:]
        h[r, rng.choice(n, size=n_top, replace=False)] = rng.choice(top, size=n_top)
    return h


def serving_batch(rows: int = 1024, vocab: int = 151936, seed: int = 4, hist: int = 256) -> Workload:
    """Config 4 (and the throughput sweep): 70 % of rows N(0, 2^2) + 16 spikes U(8, 14), 30 % near-uniform
    N(0, 0.3^2); temperature 0.7, top_k 50, top_p 0.95, min_p 0.02, repeat_penalty 1.15 over a 256-id window;
    seeds 4000 + row."""
    rng = np.random.Generator(np.random.PCG64(seed))
    x = rng.standard_normal((rows, vocab), dtype=np.float32)
    flat = rng.random(rows) < 0.30
    x[flat] *= np.float32(0.3)
    x[~flat] *= np.float32(2.0)
    _add_spikes(rng, x, 16, 8.0, 14.0, rows=np.nonzero(~flat)[0])
    params = make_params(rows, temperature=0.7, top_k=50, top_p=0.95, min_p=0.02, repeat_penalty=1.15,
                         repeat_last_n=hist, seed=4000 + np.arange(rows, dtype=np.uint64))
    history = _history(rng, x, hist)
    return Workload("serving_batch", x, params, history, np.full(rows, hist, np.int32))


def sharded_batch(rows: int = 128, vocab: int = 151936, seed: int = 5) -> Workload:
    """Config 5: N(0, 2^2) + 16 spikes U(8, 14); top_k 64 (local and global), temperature 0.9, top_p 0.9,
    min_p 0.05, no penalty; seeds 5000 + row.  The checker runs on the whole (unsharded) row."""
    rng = np.random.Generator(np.random.PCG64(seed))
    x = _normal(rng, (rows, vocab), 2.0)
    _add_spikes(rng, x, 16, 8.0, 14.0)
    params = make_params(rows, temperature=0.9, top_k=64, top_p=0.9, min_p=0.05, repeat_penalty=1.0, repeat_last_n=64,
                         seed=5000 + np.arange(rows, dtype=np.uint64))
    return Workload("sharded_batch", x, params, None, None)


def sampler_bench_row(vocab: int = 151936):
    """The reference micro-benchmark's input (bench/sampler_bench.cpp:6-7): 1000 distinct values, ~152-way ties,
    so the index tie-break decides the whole candidate set; 300 history ids of which the last 64 count."""
    i = np.arange(vocab, dtype=np.int64)
    x = (((i * 7919) % 1000).astype(np.float32) / np.float32(100.0)).reshape(1, vocab)
    h = ((np.arange(300, dtype=np.int64) * 31) % vocab).astype(np.int32).reshape(1, 300)
    return x, h
