"""A second, independent restatement of the reference sampler in plain Python.

Written from src/molla/engine/sample.mojo line by line with numpy float32 scalars
(every operation rounded on its own), the reference's own heapsort, and `exp`
taken as a parameter. It exists to cross-check the C oracle on small cases and to
generate the committed golden vectors (make_golden.py); it is far too slow for
anything else. The Mojo reference itself cannot run where this is built.
"""
from __future__ import annotations

import math

import numpy as np

F = np.float32
M64 = (1 << 64) - 1


def mix(z: int) -> int:  # sample.mojo:49-59
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & M64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & M64
    return z ^ (z >> 31)


def draw(seed: int, counter: int) -> np.float32:  # sample.mojo:62-71
    h = mix((seed ^ mix((counter + 0x9E3779B97F4A7C15) & M64)) & M64)
    return F(F(h >> 40) / F(1 << 24))


def exp_pinned(x) -> np.float32:
    """The fp32 exponential the oracle and the kernels share, restated with exact
    rational arithmetic for the fused multiply-adds (an fma rounds once)."""
    from fractions import Fraction

    x = F(x)
    if np.isnan(x):
        return x
    if x > F(88.72284):
        return F(np.inf)
    if x < F(-104.0):
        return F(0.0)

    def fma(a, b, c):
        return F(float(Fraction(float(a)) * Fraction(float(b)) + Fraction(float(c))))

    LOG2E, LN2_HI, LN2_LO, MAGIC = F(1.442695040888963), F(0.693145751953125), F(1.428606765330187e-06), F(12582912.0)
    t = fma(x, LOG2E, MAGIC)
    nf = F(t - MAGIC)
    r = fma(nf, -LN2_HI, x)
    r = fma(nf, -LN2_LO, r)
    p = F(1.0) / F(5040.0)
    for c in (F(1.0) / F(720.0), F(1.0) / F(120.0), F(1.0) / F(24.0), F(1.0) / F(6.0), F(0.5), F(1.0), F(1.0)):
        p = fma(p, r, c)
    n = int(nf)
    if n > 127:
        return F(F(p * F(2.0 ** (n - 64))) * F(2.0 ** 64))
    if n >= -126:
        return F(p * F(2.0 ** n))
    return F(F(p * F(2.0 ** (n + 64))) * F(2.0 ** -64))


class Config:  # sample.mojo:74-154
    def __init__(self, **kw):
        self.temperature = 0.0
        self.top_k = 0
        self.top_p = 1.0
        self.min_p = 0.0
        self.typical_p = 1.0
        self.repeat_penalty = 1.0
        self.frequency_penalty = 0.0
        self.presence_penalty = 0.0
        self.repeat_last_n = 64
        self.seed = 0
        for k, v in kw.items():
            setattr(self, k, v)

    def greedy(self):
        return F(self.temperature) <= 0

    def penalizing(self):
        if self.repeat_last_n <= 0:
            return False
        return F(self.repeat_penalty) != 1.0 or F(self.frequency_penalty) != 0.0 or F(self.presence_penalty) != 0.0


class Sampler:  # sample.mojo:157-594
    def __init__(self, config: Config, vocab: int, exp=exp_pinned):
        self.config = config
        self.recent = [-1] * config.repeat_last_n
        self.head = 0
        self.filled = 0
        self.ids = list(range(vocab))
        self.vals = [F(0)] * vocab
        self.kept = 0
        self.drawn = 0
        self.bias_ids, self.bias_vals = [], []
        self.exp = exp

    def vocab(self):
        return len(self.ids)

    def bias(self, token, amount):
        self.bias_ids.append(token)
        self.bias_vals.append(F(amount))

    def observe(self, token):
        if not self.recent:
            return
        self.recent[self.head] = token
        self.head = (self.head + 1) % len(self.recent)
        if self.filled < len(self.recent):
            self.filled += 1

    def count_of(self, token):
        return sum(1 for i in range(self.filled) if self.recent[i] == token)

    def logprobs(self, z):
        z = [F(v) for v in z]
        top = z[0]
        for v in z[1:]:
            if v > top:
                top = v
        s = 0.0
        for v in z:
            s += float(self.exp(F(v - top)))
        offset = F(math.log(s))
        return np.array([F(F(v - top) - offset) for v in z], dtype=F)

    def _swap(self, a, b):
        self.vals[a], self.vals[b] = self.vals[b], self.vals[a]
        self.ids[a], self.ids[b] = self.ids[b], self.ids[a]

    def _sift(self, at, n):
        root = at
        while True:
            child = root * 2 + 1
            if child >= n:
                return
            if child + 1 < n and self.vals[child + 1] > self.vals[child]:
                child += 1
            if self.vals[root] >= self.vals[child]:
                return
            self._swap(root, child)
            root = child

    def _sort(self):
        n = self.kept
        for start in range(n // 2 - 1, -1, -1):
            self._sift(start, n)
        for end in range(n - 1, 0, -1):
            self._swap(0, end)
            self._sift(0, end)
        i, j = 0, n - 1
        while i < j:
            self._swap(i, j)
            i += 1
            j -= 1

    def pick(self, row):
        c = self.config
        V = self.vocab()
        if c.greedy() and not c.penalizing() and not self.bias_ids:
            best = 0
            for i in range(1, V):
                if F(row[i]) > F(row[best]):
                    best = i
            self._took(best)
            return best
        self.ids = list(range(V))
        self.vals = [F(v) for v in row]
        self.kept = V
        for i in range(self.kept):  # _bias
            for j, t in enumerate(self.bias_ids):
                if t == self.ids[i]:
                    self.vals[i] = F(self.vals[i] + self.bias_vals[j])
        if c.penalizing():  # _penalise
            for i in range(self.kept):
                n = self.count_of(self.ids[i])
                if n == 0:
                    continue
                v = self.vals[i]
                v = F(v / F(c.repeat_penalty)) if v > 0 else F(v * F(c.repeat_penalty))
                v = F(v - F(F(n) * F(c.frequency_penalty)))
                v = F(v - F(c.presence_penalty))
                self.vals[i] = v
        self.penalised = np.array(self.vals, dtype=F)
        if c.greedy():
            best = 0
            for i in range(1, self.kept):
                if self.vals[i] > self.vals[best]:
                    best = i
            at = self.ids[best]
            self._took(at)
            return at
        t = F(c.temperature)
        if t != 1.0:
            self.vals = [F(v / t) for v in self.vals]
        top = self.vals[0]
        for v in self.vals[1:]:
            if v > top:
                top = v
        s = F(0)
        for i in range(self.kept):
            self.vals[i] = self.exp(F(self.vals[i] - top))
            s = F(s + self.vals[i])
        self.z_sum = s
        if s > 0:
            self.vals = [F(v / s) for v in self.vals]
        k = c.top_k
        if 0 < k < self.kept:
            self._sort()
            self.kept = k
        p = F(c.top_p)
        if p < 1.0 and self.kept > 1:
            self._sort()
            acc = F(0)
            for i in range(self.kept):
                acc = F(acc + self.vals[i])
                if acc >= p:
                    self.kept = i + 1
                    break
        floor_ = F(c.min_p)
        if floor_ > 0 and self.kept > 1:
            topv = max(self.vals[: self.kept])
            cut = F(topv * floor_)
            write = 0
            for i in range(self.kept):
                if self.vals[i] >= cut:
                    self._swap(write, i)
                    write += 1
            if write > 0:
                self.kept = write
        tp = F(c.typical_p)
        if tp < 1.0 and self.kept > 1:
            ent = F(0)
            for i in range(self.kept):
                if self.vals[i] > 0:
                    ent = F(ent - F(self.vals[i] * F(math.log(self.vals[i]))))
            dist = []
            for i in range(self.kept):
                sur = F(-F(math.log(self.vals[i]))) if self.vals[i] > 0 else F(0)
                d = F(sur - ent)
                dist.append(d if d >= 0 else F(-d))
            for i in range(1, self.kept):
                j = i
                while j > 0 and dist[j - 1] > dist[j]:
                    dist[j - 1], dist[j] = dist[j], dist[j - 1]
                    self._swap(j - 1, j)
                    j -= 1
            acc = F(0)
            for i in range(self.kept):
                acc = F(acc + self.vals[i])
                if acc >= tp:
                    self.kept = i + 1
                    break
        tot = F(0)
        for i in range(self.kept):
            tot = F(tot + self.vals[i])
        if tot <= 0:
            at = self.ids[0]
        else:
            target = F(draw(c.seed, self.drawn) * tot)
            acc = F(0)
            at = self.ids[self.kept - 1]
            for i in range(self.kept):
                acc = F(acc + self.vals[i])
                if target < acc:
                    at = self.ids[i]
                    break
        self._took(at)
        return at

    def _took(self, token):
        self.observe(token)
        self.drawn += 1
