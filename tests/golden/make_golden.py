"""Generates tests/golden/sampler_golden.npz from the pure-Python restatement (pyref.py).

    python tests/golden/make_golden.py

Each case is one sampler configuration over a small seeded logit row, stepped several
times so the penalty window and the draw counter move. Stored per step: the window
before the pick, the draw counter, the token, the softmax denominator and the row after
bias and penalties. The C oracle and the CUDA library are both tested against this file.
The reference (Mojo) cannot run where this is generated; the file pins the two
restatements to each other and records the reference's own numeric fixtures
(tests/test_sample.mojo:25-33, 367-372; tests/test_gpu_ops.mojo:365-407).
"""
from __future__ import annotations

import math
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
import pyref  # noqa: E402

F = np.float32


def logits_row(rng, V):
    perm = rng.permutation(V)
    return (3.0 * rng.standard_normal(V) - 1.2 * np.log1p(perm)).astype(F)


def cases():
    rng = np.random.default_rng(20260901)
    five = np.array([math.log(8), math.log(4), math.log(2), 0, 0], dtype=F)  # test_sample.mojo:25-33
    close = np.array([3.0, 2.9, 1.0, 0.0, -1.0], dtype=F)                    # test_sample.mojo:367-372
    out = []
    out.append(("five_t1", five, dict(temperature=1.0, seed=20260901), [], 20))
    out.append(("five_topk2", five, dict(temperature=1.0, top_k=2, seed=11), [], 12))
    out.append(("five_topp07", five, dict(temperature=1.0, top_p=0.7, seed=13), [], 12))
    out.append(("five_topp08", five, dict(temperature=1.0, top_p=0.8, seed=13), [], 12))
    out.append(("five_hot", five, dict(temperature=100.0, seed=5), [], 12))
    out.append(("five_cold", five, dict(temperature=0.01, seed=5), [], 6))
    out.append(("close_freq", close, dict(frequency_penalty=0.2), [], 4))
    out.append(("close_rep", close, dict(repeat_penalty=1.5, temperature=0.8, seed=3), [], 8))
    out.append(("five_bias", five, dict(temperature=2.0, seed=11), [(0, -100.0), (1, -100.0), (3, -100.0), (4, -100.0)], 4))
    out.append(("five_bias_sum", five, dict(frequency_penalty=11.0), [(2, 5.0), (2, 5.0)], 3))
    for V, cfg in ((33, dict(temperature=0.9, top_k=7, top_p=0.85, repeat_penalty=1.2, seed=7)),
                   (257, dict(temperature=1.1, top_p=0.9, presence_penalty=0.4, frequency_penalty=0.25, seed=8)),
                   (600, dict(temperature=0.7, top_k=40, top_p=0.9, repeat_penalty=1.1, seed=9)),
                   (600, dict(temperature=1.3, seed=10)),
                   (1000, dict(temperature=1.0, top_k=120, top_p=0.97, seed=12, repeat_last_n=16, frequency_penalty=0.1)),
                   (1501, dict(temperature=1.5, top_p=0.95, seed=14))):
        out.append((f"gen_V{V}_s{cfg['seed']}", logits_row(rng, V), cfg, [], 6))
    # min-p (test_sample.mojo:305-329 for the five-logit fixture), sorted and unsorted rows
    out.append(("five_minp03", five, dict(temperature=1.0, min_p=0.3, seed=17), [], 12))
    out.append(("five_minp02", five, dict(temperature=1.0, min_p=0.2, seed=17), [], 12))
    for V, cfg in ((600, dict(temperature=0.9, top_k=40, min_p=0.05, seed=21)),
                   (257, dict(temperature=1.2, min_p=0.02, seed=22)),
                   (1000, dict(temperature=1.1, top_p=0.95, min_p=0.1, seed=23, repeat_penalty=1.15))):
        out.append((f"minp_V{V}_s{cfg['seed']}", logits_row(rng, V), cfg, [], 6))
    return out


def main():
    store = {}
    names = []
    for name, row, cfg, bias, steps in cases():
        c = pyref.Config(**cfg)
        s = pyref.Sampler(c, len(row))
        for t, a in bias:
            s.bias(t, a)
        toks, zs, pens, wins, drawn = [], [], [], [], []
        for _ in range(steps):
            wins.append(list(s.recent[: s.filled]))
            drawn.append(s.drawn)
            s.z_sum = F(0)
            s.penalised = np.array(row, dtype=F)
            toks.append(s.pick(row))
            zs.append(s.z_sum)
            pens.append(s.penalised.copy())
        names.append(name)
        store[f"{name}/logits"] = row
        store[f"{name}/cfg"] = np.array([cfg.get("temperature", 0.0), cfg.get("top_k", 0), cfg.get("top_p", 1.0),
                                         cfg.get("repeat_penalty", 1.0), cfg.get("frequency_penalty", 0.0),
                                         cfg.get("presence_penalty", 0.0), cfg.get("repeat_last_n", 64),
                                         cfg.get("seed", 0), cfg.get("min_p", 0.0), cfg.get("typical_p", 1.0)],
                                        dtype=np.float64)
        store[f"{name}/bias_ids"] = np.array([b[0] for b in bias], dtype=np.int64)
        store[f"{name}/bias_vals"] = np.array([b[1] for b in bias], dtype=F)
        store[f"{name}/tokens"] = np.array(toks, dtype=np.int32)
        store[f"{name}/z_sum"] = np.array(zs, dtype=F)
        store[f"{name}/penalised"] = np.stack(pens)
        store[f"{name}/drawn"] = np.array(drawn, dtype=np.uint64)
        width = max(1, max(len(w) for w in wins))
        win = np.full((steps, width), -1, dtype=np.int64)
        for i, w in enumerate(wins):
            win[i, : len(w)] = w
        store[f"{name}/windows"] = win
        store[f"{name}/window_len"] = np.array([len(w) for w in wins], dtype=np.int32)
        store[f"{name}/logprobs"] = s.logprobs(row)
    store["names"] = np.array(names)
    # the pinned exponential on a spread of arguments
    xs = np.concatenate([np.linspace(-104.5, 0, 4001), -np.logspace(-8, 2, 400), [0.0, -0.0, -87.3365, -103.97, 1.0, 88.0]]).astype(F)
    store["exp_x"] = xs
    store["exp_y"] = np.array([pyref.exp_pinned(x) for x in xs], dtype=F)
    # draw() known answers
    pairs = [(0, 0), (1, 0), (1, 1), (1, 7), (2, 0), (99, 0), (99, 255), (20260901, 0), (20260901, 19), (4242, 0),
             (777, 11), (2**64 - 1, 2**64 - 1)]
    store["draw_seed"] = np.array([p[0] for p in pairs], dtype=np.uint64)
    store["draw_counter"] = np.array([p[1] for p in pairs], dtype=np.uint64)
    store["draw_value"] = np.array([pyref.draw(*p) for p in pairs], dtype=F)
    np.savez_compressed(os.path.join(HERE, "sampler_golden.npz"), **store)
    print("wrote", len(names), "cases")


if __name__ == "__main__":
    main()
