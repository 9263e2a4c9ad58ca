"""Seeded synthetic sampler workloads.

The reference publishes no benchmark inputs for its sampler, so every workload
here is generated: logits are `3.0*N(0,1) - 1.2*ln(1 + perm(i))` with a seeded
permutation of the vocabulary per row (a heavy head over a long noisy tail, the
shape of a language-model logit row), computed in fp64 and rounded to fp32.
Histories, per-row parameters, seeds and draw counters are seeded as well, so
the CPU checker and the GPU library always see identical inputs.

A workload is a plain dict of numpy arrays in the layout the batched sampler
entry point takes: per-row parameter arrays of length B, `hist`/`hist_off` as a
ragged list of penalty windows, `bias_*` likewise.
"""
from __future__ import annotations

import numpy as np


def make_logits(B: int, V: int, seed: int, boost: int = 0, boost_by: float = 12.0) -> np.ndarray:
    rng = np.random.default_rng(seed)
    out = np.empty((B, V), dtype=np.float32)
    ranks = np.log1p(np.arange(V, dtype=np.float64)) * 1.2
    for r in range(B):
        perm = rng.permutation(V)
        row = 3.0 * rng.standard_normal(V) - ranks[perm]
        if boost > 0:
            row[rng.choice(V, size=boost, replace=False)] += boost_by
        out[r] = row.astype(np.float32)
    return out


def _uniform_hist(rng, B, V, H):
    hist = rng.integers(0, V, size=(B, H), dtype=np.int64).reshape(-1)
    off = (np.arange(B + 1, dtype=np.int64) * H).astype(np.int32)
    return hist, off


def _zipf_hist(rng, B, V, H, s=1.1):
    w = np.arange(1, V + 1, dtype=np.float64) ** (-s)
    cdf = np.cumsum(w)
    cdf /= cdf[-1]
    hist = np.empty((B, H), dtype=np.int64)
    for r in range(B):
        ids = rng.permutation(V)
        ranks = np.searchsorted(cdf, rng.random(H), side="left")
        hist[r] = ids[np.minimum(ranks, V - 1)]
    off = (np.arange(B + 1, dtype=np.int64) * H).astype(np.int32)
    return hist.reshape(-1), off


def _base(B, V, seed):
    return dict(
        B=B, V=V,
        temperature=np.zeros(B, np.float32), top_k=np.zeros(B, np.int32),
        top_p=np.ones(B, np.float32), min_p=np.zeros(B, np.float32),
        typical_p=np.ones(B, np.float32), repeat_penalty=np.ones(B, np.float32),
        frequency_penalty=np.zeros(B, np.float32), presence_penalty=np.zeros(B, np.float32),
        seed=(np.uint64(seed) + np.arange(B, dtype=np.uint64)),
        drawn=(np.arange(B, dtype=np.uint64) % np.uint64(4)),
        hist=np.zeros(0, np.int64), hist_off=np.zeros(B + 1, np.int32),
        window_on=np.ones(B, np.uint8),
        bias_ids=np.zeros(0, np.int64), bias_vals=np.zeros(0, np.float32),
        bias_off=np.zeros(B + 1, np.int32), top_n=0,
    )


def config1(seed: int = 1001, B: int = 1, V: int = 32000):
    """One row, V=32000: temp 0.7, top-k 40, top-p 0.9, repetition penalty 1.1 over 64 ids."""
    rng = np.random.default_rng(seed + 7)
    w = _base(B, V, seed)
    w["name"] = f"c1:B={B},V={V},temp0.7,topk40,topp0.9,rep1.1,H=64"
    w["logits"] = make_logits(B, V, seed)
    w["temperature"][:] = 0.7
    w["top_k"][:] = 40
    w["top_p"][:] = 0.9
    w["repeat_penalty"][:] = 1.1
    w["hist"], w["hist_off"] = _uniform_hist(rng, B, V, 64)
    return w


def config2(seed: int = 2002, B: int = 64, V: int = 151936, H: int = 512):
    """B=64: temp 1.0, top-p 0.95, presence 0.5 + frequency 0.3 over Zipf windows, top-5 logprobs."""
    rng = np.random.default_rng(seed + 7)
    w = _base(B, V, seed)
    w["name"] = f"c2:B={B},V={V},temp1.0,topp0.95,pres0.5,freq0.3,H={H},top5"
    w["logits"] = make_logits(B, V, seed)
    w["temperature"][:] = 1.0
    w["top_p"][:] = 0.95
    w["presence_penalty"][:] = 0.5
    w["frequency_penalty"][:] = 0.3
    w["hist"], w["hist_off"] = _zipf_hist(rng, B, V, H)
    w["top_n"] = 5
    return w


def config3(seed: int = 3003, B: int = 256, V: int = 151936, H: int = 256):
    """B=256, per-row parameters: temp U[0,1.5] (every 16th row exactly 0 = greedy),
    top-k from {0,1,20,50,100}, top-p U[0.5,1.0], repetition penalty U[1.0,1.3]."""
    rng = np.random.default_rng(seed + 7)
    w = _base(B, V, seed)
    w["name"] = f"c3:B={B},V={V},hetero,H={H}"
    w["logits"] = make_logits(B, V, seed)
    t = rng.uniform(0.0, 1.5, B).astype(np.float32)
    t[::16] = 0.0
    w["temperature"][:] = t
    w["top_k"][:] = rng.choice(np.array([0, 1, 20, 50, 100], np.int32), size=B)
    p = rng.uniform(0.5, 1.0, B).astype(np.float32)
    w["top_p"][:] = np.minimum(p, np.float32(1.0))
    w["repeat_penalty"][:] = rng.uniform(1.0, 1.3, B).astype(np.float32)
    w["hist"], w["hist_off"] = _uniform_hist(rng, B, V, H)
    return w


def config4(seed: int = 4004, B: int = 1024, V: int = 262144):
    """Large-k stress: top-k 1024, top-p 0.99, temp 0.9, eight tokens per row boosted by +12."""
    w = _base(B, V, seed)
    w["name"] = f"c4:B={B},V={V},topk1024,topp0.99,temp0.9,boost8"
    w["logits"] = make_logits(B, V, seed, boost=8)
    w["temperature"][:] = 0.9
    w["top_k"][:] = 1024
    w["top_p"][:] = 0.99
    w["window_on"][:] = 0
    return w


def config5(seed: int = 5005, B: int = 128, V: int = 151936, H: int = 128):
    """Vocab-sharded case (8 slices of 18992): top-k 50, top-p 0.9, temp 0.8, rep 1.1."""
    rng = np.random.default_rng(seed + 7)
    w = _base(B, V, seed)
    w["name"] = f"c5:B={B},V={V},topk50,topp0.9,temp0.8,rep1.1,H={H},vocab-sharded"
    w["logits"] = make_logits(B, V, seed)
    w["temperature"][:] = 0.8
    w["top_k"][:] = 50
    w["top_p"][:] = 0.9
    w["repeat_penalty"][:] = 1.1
    w["hist"], w["hist_off"] = _uniform_hist(rng, B, V, H)
    return w


def slice_rows(w: dict, lo: int, hi: int) -> dict:
    """Rows [lo, hi) of a workload: the shard one GPU takes in row-sharded mode."""
    out = dict(w)
    out["B"] = hi - lo
    out["logits"] = w["logits"][lo:hi]
    for k in ("temperature", "top_k", "top_p", "min_p", "typical_p", "repeat_penalty",
              "frequency_penalty", "presence_penalty", "seed", "drawn", "window_on"):
        out[k] = w[k][lo:hi]
    for ids, vals, off in (("hist", None, "hist_off"), ("bias_ids", "bias_vals", "bias_off")):
        o = w[off].astype(np.int64)
        out[ids] = w[ids][o[lo]:o[hi]]
        if vals:
            out[vals] = w[vals][o[lo]:o[hi]]
        out[off] = (o[lo:hi + 1] - o[lo]).astype(np.int32)
    return out


SAMPLER_KEYS = ("temperature", "top_k", "top_p", "min_p", "typical_p", "repeat_penalty",
                "frequency_penalty", "presence_penalty", "seed", "drawn", "hist", "hist_off",
                "window_on", "bias_ids", "bias_vals", "bias_off")
