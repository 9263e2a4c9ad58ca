"""Shared helpers of the test-suite: an oracle-backed sampler with the reference's
per-sequence interface, and the golden-case reader."""
from __future__ import annotations

import numpy as np


class OracleSampler:
    """`Sampler` of src/molla/engine/sample.mojo over the C oracle: keeps the ring window
    and the draw counter on the Python side and asks the oracle for one pick at a time."""

    def __init__(self, O, vocab, temperature=0.0, top_k=0, top_p=1.0, min_p=0.0, typical_p=1.0,
                 repeat_penalty=1.0, frequency_penalty=0.0, presence_penalty=0.0, repeat_last_n=64, seed=0):
        self.O = O
        self.V = vocab
        self.cfg = dict(temperature=temperature, top_k=top_k, top_p=top_p, min_p=min_p, typical_p=typical_p,
                        repeat_penalty=repeat_penalty, frequency_penalty=frequency_penalty,
                        presence_penalty=presence_penalty)
        self.seed = seed
        self.recent = [-1] * repeat_last_n
        self.head = 0
        self.filled = 0
        self.drawn = 0
        self.bias_ids, self.bias_vals = [], []

    def bias(self, t, a):
        self.bias_ids.append(t)
        self.bias_vals.append(a)

    def observe(self, token):
        if not self.recent:
            return
        self.recent[self.head] = token
        self.head = (self.head + 1) % len(self.recent)
        self.filled = min(self.filled + 1, len(self.recent))

    def count_of(self, token):
        return sum(1 for i in range(self.filled) if self.recent[i] == token)

    def reset(self):
        self.head = self.filled = self.drawn = 0

    def pick(self, logits, row=0):
        logits = np.asarray(logits, np.float32)
        if logits.ndim == 1:
            logits = logits[None, :]
        hist = np.array(self.recent[: self.filled], np.int64)
        r = self.O.pick_batch(
            logits[row:row + 1], **self.cfg, seed=self.seed, drawn=self.drawn, hist=hist,
            hist_off=np.array([0, len(hist)], np.int32), window_on=np.array([1 if self.recent else 0], np.uint8),
            bias_ids=np.array(self.bias_ids, np.int64), bias_vals=np.array(self.bias_vals, np.float32),
            bias_off=np.array([0, len(self.bias_ids)], np.int32), nthreads=1)
        t = int(r["tokens"][0])
        self.observe(t)
        self.drawn += 1
        return t


def golden_case(g, name):
    cfg = g[f"{name}/cfg"]
    return dict(
        logits=g[f"{name}/logits"], temperature=np.float32(cfg[0]), top_k=int(cfg[1]), top_p=np.float32(cfg[2]),
        repeat_penalty=np.float32(cfg[3]), frequency_penalty=np.float32(cfg[4]), presence_penalty=np.float32(cfg[5]),
        repeat_last_n=int(cfg[6]), seed=int(cfg[7]), min_p=np.float32(cfg[8]), typical_p=np.float32(cfg[9]), bias_ids=g[f"{name}/bias_ids"], bias_vals=g[f"{name}/bias_vals"],
        tokens=g[f"{name}/tokens"], z_sum=g[f"{name}/z_sum"], penalised=g[f"{name}/penalised"],
        drawn=g[f"{name}/drawn"], windows=g[f"{name}/windows"], window_len=g[f"{name}/window_len"],
        logprobs=g[f"{name}/logprobs"])


def golden_as_batch(g, name):
    """One golden case (several steps of one sampler) as a batch: one row per step."""
    c = golden_case(g, name)
    steps = len(c["tokens"])
    V = len(c["logits"])
    w = dict(B=steps, V=V, logits=np.repeat(c["logits"][None, :], steps, 0))
    full = lambda v, dt: np.full(steps, v, dtype=dt)
    w.update(temperature=full(c["temperature"], np.float32), top_k=full(c["top_k"], np.int32),
             top_p=full(c["top_p"], np.float32), min_p=full(c["min_p"], np.float32), typical_p=full(c["typical_p"], np.float32),
             repeat_penalty=full(c["repeat_penalty"], np.float32),
             frequency_penalty=full(c["frequency_penalty"], np.float32),
             presence_penalty=full(c["presence_penalty"], np.float32),
             window_on=full(1 if c["repeat_last_n"] > 0 else 0, np.uint8),
             seed=full(c["seed"], np.uint64), drawn=c["drawn"].astype(np.uint64))
    hist, off = [], [0]
    for i in range(steps):
        hist.extend(c["windows"][i, : c["window_len"][i]].tolist())
        off.append(len(hist))
    w["hist"] = np.array(hist, np.int64)
    w["hist_off"] = np.array(off, np.int32)
    nb = len(c["bias_ids"])
    w["bias_ids"] = np.tile(c["bias_ids"], steps).astype(np.int64)
    w["bias_vals"] = np.tile(c["bias_vals"], steps).astype(np.float32)
    w["bias_off"] = (np.arange(steps + 1) * nb).astype(np.int32)
    return w, c
