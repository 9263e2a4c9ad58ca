"""Host side of the sampler: the reference's `SamplerConfig` / `Sampler` interface
(src/molla/engine/sample.mojo:74-363) over the CUDA library.

A `Sampler` keeps what the reference's keeps per sequence - the settings, the
penalty window as a ring, the draw counter, the logit-bias list - and nothing
else: the candidate arrays the reference owns (`ids`, `vals`) live on the device
for the length of one call. `pick` samples one row; `pick_rows` is the batched
form that replaces the per-row loop of the decode step
(src/molla/engine/batch.mojo:503-519) with one launch.

PyTorch is used for device memory and streams only.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, replace
from typing import Iterable, Sequence

import numpy as np
import torch

from . import capi

GREEDY = 0.0
_F32 = np.float32


@dataclass
class SamplerConfig:
    """What a request asked for; every field's off value is its default
    (sample.mojo:74-126)."""
    temperature: float = GREEDY
    top_k: int = 0
    top_p: float = 1.0
    min_p: float = 0.0
    typical_p: float = 1.0
    repeat_penalty: float = 1.0
    frequency_penalty: float = 0.0
    presence_penalty: float = 0.0
    repeat_last_n: int = 64
    seed: int = 0

    def copy(self) -> "SamplerConfig":
        return replace(self)

    def greedy(self) -> bool:
        return _F32(self.temperature) <= 0

    def penalizing(self) -> bool:
        if self.repeat_last_n <= 0:
            return False
        return (_F32(self.repeat_penalty) != 1.0 or _F32(self.frequency_penalty) != 0.0
                or _F32(self.presence_penalty) != 0.0)

    def check(self) -> None:
        """The reference's validation rules and messages (sample.mojo:140-154)."""
        if not (_F32(self.temperature) >= 0):
            raise ValueError("a temperature cannot be negative")
        if self.top_k < 0:
            raise ValueError("a top-k cannot be negative")
        if not (0 < _F32(self.top_p) <= 1):
            raise ValueError("a top-p has to be above zero and at most one")
        if not (0 <= _F32(self.min_p) <= 1):
            raise ValueError("a min-p has to be between zero and one")
        if not (0 < _F32(self.typical_p) <= 1):
            raise ValueError("a typical-p has to be above zero and at most one")
        if not (_F32(self.repeat_penalty) > 0):
            raise ValueError("a repetition penalty of zero or less erases a logit")
        if self.repeat_last_n < 0:
            raise ValueError("a penalty window cannot be negative")


def draw(seed: int, counter: int) -> float:
    """A uniform float in [0, 1) from a seed and a counter (sample.mojo:62-71)."""
    return capi.draw(seed, counter)


def _ptr(t):
    return None if t is None else C.c_void_p(t.data_ptr())


def _stream_ptr(device) -> C.c_void_p:
    return C.c_void_p(torch.cuda.current_stream(device).cuda_stream)


class Workspace:
    """Device scratch for the batched call, sized by the library's own query."""

    def __init__(self, B: int, V: int, top_n: int, device):
        n = capi.lib().molla_sample_workspace_bytes(B, V, top_n)
        if n < 0:
            raise capi.MollaSampleError(int(n), capi.last_error())
        self.bytes = int(n)
        self.buf = torch.zeros(self.bytes, dtype=torch.uint8, device=device)


def sample_batch(logits: torch.Tensor, p: dict, top_n: int = 0, want_logprob: bool = False,
                 want_diag: bool = False, workspace: Workspace | None = None, out: dict | None = None):
    """One launch over a device-resident [B, V] fp32 block.

    `p` maps the per-row parameter names of the C entry point to device tensors
    (see `upload_params`). Returns a dict of device tensors: tokens, row_status and,
    when asked for, chosen_logprob, top_ids, top_logprobs, diag. Asynchronous on the
    current stream.
    """
    if not logits.is_cuda or logits.dtype != torch.float32 or logits.dim() != 2:
        raise ValueError("logits must be a 2-D fp32 CUDA tensor")
    if logits.stride(1) != 1:
        raise ValueError("logit rows must be contiguous")
    B, V = logits.shape
    dev = logits.device
    if B == 0:  # nothing to sample: the C entry point would be handed null pointers
        e = lambda *shape, dt=torch.float32: torch.empty(shape, dtype=dt, device=dev)
        return dict(tokens=e(0, dt=torch.int32), row_status=e(0, dt=torch.int32), chosen_logprob=e(0),
                    top_ids=e(0, top_n, dt=torch.int32), top_logprobs=e(0, top_n), diag=e(0, 4))
    if workspace is None:
        workspace = Workspace(B, V, top_n, dev)
    if out is None:
        out = {}
    tokens = out.get("tokens")
    if tokens is None:
        tokens = torch.empty(B, dtype=torch.int32, device=dev)
    status = out.get("row_status")
    if status is None:
        status = torch.empty(B, dtype=torch.int32, device=dev)
    chosen = out.get("chosen_logprob")
    if chosen is None and want_logprob:
        chosen = torch.empty(B, dtype=torch.float32, device=dev)
    top_ids = out.get("top_ids")
    top_lps = out.get("top_logprobs")
    if top_n > 0 and top_ids is None:
        top_ids = torch.empty((B, top_n), dtype=torch.int32, device=dev)
        top_lps = torch.empty((B, top_n), dtype=torch.float32, device=dev)
    diag = out.get("diag")
    if diag is None and want_diag:
        diag = torch.empty((B, 4), dtype=torch.float32, device=dev)
    g = p.get
    mask = g("mask")   # optional grammar mask: [B, ceil(V / 32)] int32 words, bit t of a row = token t allowed
    if mask is not None and (mask.dim() != 2 or mask.shape[0] != B or mask.stride(1) != 1 or mask.element_size() != 4):
        raise ValueError("the grammar mask is a [B, ceil(V/32)] tensor of 32-bit words")
    rc = capi.lib().molla_sample_batch_masked(
        _ptr(mask), mask.stride(0) if mask is not None else 0, _ptr(logits), logits.stride(0), B, V,
        _ptr(g("temperature")), _ptr(g("top_k")), _ptr(g("top_p")), _ptr(g("min_p")),
        _ptr(g("typical_p")), _ptr(g("repeat_penalty")), _ptr(g("frequency_penalty")),
        _ptr(g("presence_penalty")), _ptr(g("window_on")), _ptr(g("seed")), _ptr(g("drawn")),
        _ptr(g("hist")), _ptr(g("hist_off")), _ptr(g("bias_ids")), _ptr(g("bias_vals")),
        _ptr(g("bias_off")), top_n, _ptr(workspace.buf), workspace.bytes, _stream_ptr(dev),
        _ptr(tokens), _ptr(chosen), _ptr(top_ids), _ptr(top_lps), _ptr(status), _ptr(diag))
    capi.check(rc)
    return dict(tokens=tokens, row_status=status, chosen_logprob=chosen, top_ids=top_ids,
                top_logprobs=top_lps, diag=diag)


class HostBlock:
    """Host-resident inputs and outputs for `sample_batch_host`: the logit block and the
    per-row parameters in pinned memory (what the reference's decode loop holds after
    `copy_out`), plus the device workspace the call stages them in."""

    def __init__(self, w: dict, device, top_n: int = 0, want_logprob: bool = False):
        self.B, self.V = w["logits"].shape
        self.device = torch.device(device)
        self.top_n = top_n
        self.logits = torch.from_numpy(np.ascontiguousarray(w["logits"], np.float32)).pin_memory()
        self.p = {}
        for k, dt in _PARAM_DTYPES.items():
            if k in w and w[k] is not None:
                a = np.ascontiguousarray(w[k], dtype=dt)
                if dt == np.uint64:
                    a = a.view(np.int64)
                if a.size == 0:
                    a = np.zeros(1, a.dtype)
                self.p[k] = torch.from_numpy(a.copy()).pin_memory()
        n_hist = int(w["hist_off"][-1]) if "hist_off" in w else 0
        n_bias = int(w["bias_off"][-1]) if "bias_off" in w else 0
        n = capi.lib().molla_sample_host_workspace_bytes(self.B, self.V, n_hist, n_bias, top_n)
        if n < 0:
            raise capi.MollaSampleError(int(n), capi.last_error())
        self.ws_bytes = int(n)
        self.ws = torch.zeros(self.ws_bytes, dtype=torch.uint8, device=self.device)
        self.tokens = torch.empty(self.B, dtype=torch.int32).pin_memory()
        self.status = torch.empty(self.B, dtype=torch.int32).pin_memory()
        self.chosen = torch.empty(self.B, dtype=torch.float32).pin_memory() if want_logprob else None
        self.top_ids = torch.empty((self.B, max(top_n, 1)), dtype=torch.int32).pin_memory() if top_n else None
        self.top_lps = torch.empty((self.B, max(top_n, 1)), dtype=torch.float32).pin_memory() if top_n else None
        self.h2d_bytes = self.logits.numel() * 4 + sum(t.numel() * t.element_size() for t in self.p.values())
        self.d2h_bytes = self.B * 8 + (self.B * 4 if want_logprob else 0) + self.B * top_n * 8


def sample_batch_host(hb: HostBlock) -> None:
    """Host block in, host tokens out: copies, launch and copies back in one synchronous
    C call (`molla_sample_batch_host`). Results land in hb.tokens / hb.status / ..."""
    g = hb.p.get
    rc = capi.lib().molla_sample_batch_host(
        _ptr(hb.logits), hb.V, hb.B, hb.V,
        _ptr(g("temperature")), _ptr(g("top_k")), _ptr(g("top_p")), _ptr(g("min_p")),
        _ptr(g("typical_p")), _ptr(g("repeat_penalty")), _ptr(g("frequency_penalty")),
        _ptr(g("presence_penalty")), _ptr(g("window_on")), _ptr(g("seed")), _ptr(g("drawn")),
        _ptr(g("hist")), _ptr(g("hist_off")), _ptr(g("bias_ids")), _ptr(g("bias_vals")),
        _ptr(g("bias_off")), hb.top_n, _ptr(hb.ws), hb.ws_bytes, _stream_ptr(hb.device),
        _ptr(hb.tokens), _ptr(hb.chosen), _ptr(hb.top_ids), _ptr(hb.top_lps), _ptr(hb.status))
    capi.check(rc)


def penalised(logits: torch.Tensor, p: dict, workspace: Workspace | None = None) -> torch.Tensor:
    """The block after logit bias and penalties, before temperature (sample.mojo:381-417)."""
    B, V = logits.shape
    dev = logits.device
    if workspace is None:
        workspace = Workspace(B, V, 0, dev)
    out = torch.empty((B, V), dtype=torch.float32, device=dev)
    g = p.get
    rc = capi.lib().molla_sample_penalised(
        _ptr(logits), logits.stride(0), B, V, _ptr(g("repeat_penalty")),
        _ptr(g("frequency_penalty")), _ptr(g("presence_penalty")), _ptr(g("window_on")),
        _ptr(g("hist")), _ptr(g("hist_off")), _ptr(g("bias_ids")), _ptr(g("bias_vals")),
        _ptr(g("bias_off")), _ptr(workspace.buf), workspace.bytes, _stream_ptr(dev), _ptr(out))
    capi.check(rc)
    return out


def logprobs_block(logits: torch.Tensor) -> torch.Tensor:
    """`Sampler.logprobs` (sample.mojo:268-293) for every row of a device block."""
    B, V = logits.shape
    out = torch.empty((B, V), dtype=torch.float32, device=logits.device)
    capi.check(capi.lib().molla_sample_logprobs(_ptr(logits), logits.stride(0), B, V,
                                                _stream_ptr(logits.device), _ptr(out)))
    return out


def expf_device(x: torch.Tensor) -> torch.Tensor:
    out = torch.empty_like(x)
    capi.check(capi.lib().molla_sample_expf(_ptr(x), x.numel(), _stream_ptr(x.device), _ptr(out)))
    return out


def logf_device(x: torch.Tensor) -> torch.Tensor:
    out = torch.empty_like(x)
    capi.check(capi.lib().molla_sample_logf(_ptr(x), x.numel(), _stream_ptr(x.device), _ptr(out)))
    return out


_PARAM_DTYPES = dict(
    temperature=np.float32, top_k=np.int32, top_p=np.float32, min_p=np.float32,
    typical_p=np.float32, repeat_penalty=np.float32, frequency_penalty=np.float32,
    presence_penalty=np.float32, window_on=np.uint8, seed=np.uint64, drawn=np.uint64,
    hist=np.int64, hist_off=np.int32, bias_ids=np.int64, bias_vals=np.float32, bias_off=np.int32,
)


def upload_params(w: dict, device, pinned: bool = False) -> dict:
    """Per-row parameter arrays (numpy, as a workload dict holds them) -> device tensors."""
    out = {}
    for k, dt in _PARAM_DTYPES.items():
        if k not in w or w[k] is None:
            continue
        a = np.ascontiguousarray(w[k], dtype=dt)
        if dt == np.uint64:  # torch has no arithmetic on uint64; the bits are what matter
            a = a.view(np.int64)
        t = torch.from_numpy(a.copy())
        if pinned:
            t = t.pin_memory()
        out[k] = t.to(device, non_blocking=pinned)
    if "hist" in out and out["hist"].numel() == 0:
        out["hist"] = torch.zeros(1, dtype=torch.int64, device=device)
    if "bias_ids" in out and out["bias_ids"].numel() == 0:
        out["bias_ids"] = torch.zeros(1, dtype=torch.int64, device=device)
        out["bias_vals"] = torch.zeros(1, dtype=torch.float32, device=device)
    return out


class Sampler:
    """One sequence's sampler: its settings, its recent tokens, its counter
    (sample.mojo:157-363)."""

    def __init__(self, config: SamplerConfig, vocab: int, device="cuda:0"):
        config.check()
        if vocab <= 0:
            raise ValueError("a sampler needs a vocabulary")
        self.config = config.copy()
        self._vocab = int(vocab)
        self.recent = [-1] * config.repeat_last_n
        self.head = 0
        self.filled = 0
        self.drawn = 0
        self.bias_ids: list[int] = []
        self.bias_vals: list[float] = []
        self.device = torch.device(device)
        self.last_status = 0

    def vocab(self) -> int:
        return self._vocab

    def bias(self, token: int, amount: float) -> None:
        if token < 0 or token >= self._vocab:
            raise ValueError(f"a logit bias names token {token} and the vocabulary is "
                             f"{self._vocab} wide")
        self.bias_ids.append(int(token))
        self.bias_vals.append(float(amount))

    def biasing(self) -> bool:
        return len(self.bias_ids) > 0

    def reset(self) -> None:
        self.head = 0
        self.filled = 0
        self.drawn = 0

    def observe(self, token: int) -> None:
        if len(self.recent) == 0:
            return
        self.recent[self.head] = int(token)
        self.head = (self.head + 1) % len(self.recent)
        if self.filled < len(self.recent):
            self.filled += 1

    def count_of(self, token: int) -> int:
        return sum(1 for i in range(self.filled) if self.recent[i] == token)

    def _took(self, token: int) -> None:
        self.observe(token)
        self.drawn += 1

    def logprobs(self, logits: torch.Tensor) -> torch.Tensor:
        """log-softmax of the logits as the model gave them (sample.mojo:268-293). The
        reference takes an output list of exactly the block's size; here the result is
        returned, one row per row of `logits`."""
        block = logits if logits.dim() == 2 else logits[None, :]
        return logprobs_block(block)

    def pick(self, logits: torch.Tensor, row: int = 0) -> int:
        return pick_rows(logits, [self], [row])[0]


def _check_block(logits: torch.Tensor, samplers: Sequence[Sampler], rows: Sequence[int]):
    block = logits if logits.dim() == 2 else logits[None, :]
    for s, r in zip(samplers, rows):
        if block.shape[1] != s.vocab():
            raise ValueError(f"the sampler was built for a vocabulary of {s.vocab()} and got "
                             f"{block.shape[1]} logits")
        if r < 0 or r >= block.shape[0]:
            raise ValueError(f"asked for the logits of sequence {r} out of a buffer holding "
                             f"{block.shape[0]}")
    return block


def params_of(samplers: Sequence[Sampler]) -> dict:
    """The samplers' state as the parallel arrays the C entry point takes."""
    n = len(samplers)
    w = dict(
        temperature=np.array([s.config.temperature for s in samplers], np.float32),
        top_k=np.array([min(s.config.top_k, 2**31 - 1) for s in samplers], np.int32),
        top_p=np.array([s.config.top_p for s in samplers], np.float32),
        min_p=np.array([s.config.min_p for s in samplers], np.float32),
        typical_p=np.array([s.config.typical_p for s in samplers], np.float32),
        repeat_penalty=np.array([s.config.repeat_penalty for s in samplers], np.float32),
        frequency_penalty=np.array([s.config.frequency_penalty for s in samplers], np.float32),
        presence_penalty=np.array([s.config.presence_penalty for s in samplers], np.float32),
        window_on=np.array([1 if s.config.repeat_last_n > 0 else 0 for s in samplers], np.uint8),
        seed=np.array([s.config.seed & (2**64 - 1) for s in samplers], np.uint64),
        drawn=np.array([s.drawn & (2**64 - 1) for s in samplers], np.uint64),
    )
    hist, off = [], [0]
    for s in samplers:
        hist.extend(s.recent[: s.filled])
        off.append(len(hist))
    w["hist"] = np.array(hist, np.int64)
    w["hist_off"] = np.array(off, np.int32)
    bi, bv, boff = [], [], [0]
    for s in samplers:
        bi.extend(s.bias_ids)
        bv.extend(s.bias_vals)
        boff.append(len(bi))
    w["bias_ids"] = np.array(bi, np.int64)
    w["bias_vals"] = np.array(bv, np.float32)
    w["bias_off"] = np.array(boff, np.int32)
    assert len(w["temperature"]) == n
    return w


def pick_rows(logits: torch.Tensor, samplers: Sequence[Sampler], rows: Iterable[int] | None = None):
    """Sample row `rows[i]` of `logits` with `samplers[i]`, all in one launch, then record
    each token in its sampler (`_took`, sample.mojo:361-363). The batched counterpart of
    the loop at batch.mojo:509-511. Returns the tokens as a list of ints."""
    samplers = list(samplers)
    rows = list(range(len(samplers))) if rows is None else list(rows)
    block = _check_block(logits, samplers, rows)
    if not samplers:
        return []
    dev = block.device
    if rows == list(range(block.shape[0])):
        sel = block
    else:
        sel = block.index_select(0, torch.tensor(rows, device=dev))
    p = upload_params(params_of(samplers), dev)
    res = sample_batch(sel, p)
    toks = res["tokens"].cpu().tolist()
    stat = res["row_status"].cpu().tolist()
    for s, t, st in zip(samplers, toks, stat):
        s.last_status = st & 0xFFFFFFFF
        if st & capi.ROW_UNSUPPORTED:
            raise NotImplementedError("this combination of settings is not implemented on the device "
                                      "(typical_p needs top_k or top_p to leave a set inside the sorted head)")
        if st & capi.ROW_ERROR_BITS:
            raise capi.MollaSampleError(capi.ERR_DEVICE, f"row status {st:#x}")
        s._took(t)
    return toks


class DeviceSamplers:
    """The samplers of `n_slots` live sequences kept on the device: settings, recent-token
    windows and draw counters (`Sampler`'s fields, sample.mojo:157-212), so that a decode step
    samples, records the token and advances the counter without a host round trip
    (`molla_sample_decode_step`). A sequence takes a slot with `assign` and keeps it until
    another `assign` gives the slot away."""

    def __init__(self, n_slots: int, vocab: int, ring_cap: int = 64, device="cuda:0"):
        if n_slots <= 0 or vocab <= 0 or ring_cap <= 0:
            raise ValueError("slots, vocabulary and window capacity have to be positive")
        self.n_slots, self.vocab, self.ring_cap = int(n_slots), int(vocab), int(ring_cap)
        self.device = dev = torch.device(device)
        z = lambda dt, *shape: torch.zeros(shape, dtype=dt, device=dev)
        S = self.n_slots
        self.temperature = z(torch.float32, S)
        self.top_k = z(torch.int32, S)
        self.top_p = torch.ones(S, dtype=torch.float32, device=dev)
        self.min_p = z(torch.float32, S)
        self.typical_p = torch.ones(S, dtype=torch.float32, device=dev)
        self.repeat_penalty = torch.ones(S, dtype=torch.float32, device=dev)
        self.frequency_penalty = z(torch.float32, S)
        self.presence_penalty = z(torch.float32, S)
        self.seed = z(torch.int64, S)          # uint64 bit patterns
        self.drawn = z(torch.int64, S)
        self.ring = torch.full((S, self.ring_cap), -1, dtype=torch.int64, device=dev)
        self.ring_head = z(torch.int32, S)
        self.ring_filled = z(torch.int32, S)
        self.ring_len = z(torch.int32, S)
        self.stop_token = torch.full((S,), -1, dtype=torch.int64, device=dev)
        self._bias: list[list[tuple[int, float]]] = [[] for _ in range(S)]
        self._bias_dev = None
        self._ws: Workspace | None = None

    def assign(self, slot: int, config: SamplerConfig, stop_token: int = -1,
               bias: Sequence[tuple[int, float]] = ()) -> None:
        """A new sequence in `slot`: its settings, an empty window, counter zero
        (`Sampler.__init__`, sample.mojo:194-212)."""
        config.check()
        if not 0 <= slot < self.n_slots:
            raise ValueError("no such slot")
        if config.repeat_last_n > self.ring_cap:
            raise ValueError("the window is longer than the capacity these samplers were built with")
        for t, _ in bias:
            if t < 0 or t >= self.vocab:
                raise ValueError(f"a logit bias names token {t} and the vocabulary is {self.vocab} wide")
        s = int(config.seed) & (2**64 - 1)
        vals = dict(temperature=config.temperature, top_k=config.top_k, top_p=config.top_p, min_p=config.min_p,
                    typical_p=config.typical_p, repeat_penalty=config.repeat_penalty,
                    frequency_penalty=config.frequency_penalty, presence_penalty=config.presence_penalty,
                    seed=s - 2**64 if s >= 2**63 else s, drawn=0, ring_head=0, ring_filled=0,
                    ring_len=config.repeat_last_n,
                    stop_token=int(stop_token))
        for k, v in vals.items():
            getattr(self, k)[slot] = v
        self.ring[slot].fill_(-1)
        self._bias[slot] = [(int(t), float(v)) for t, v in bias]
        self._bias_dev = None

    def _bias_arrays(self):
        if self._bias_dev is None:
            ids, vals, off = [], [], [0]
            for lst in self._bias:
                ids += [t for t, _ in lst]
                vals += [v for _, v in lst]
                off.append(len(ids))
            if ids:
                dev = self.device
                self._bias_dev = (torch.tensor(ids, dtype=torch.int64, device=dev),
                                  torch.tensor(vals, dtype=torch.float32, device=dev),
                                  torch.tensor(off, dtype=torch.int32, device=dev))
            else:
                self._bias_dev = (None, None, None)
        return self._bias_dev

    def step(self, logits: torch.Tensor, rows: torch.Tensor | None, slots: torch.Tensor | None,
             final_softcap: float = 0.0, top_n: int = 0, want_logprob: bool = False) -> dict:
        """One decode step: batch row r samples logit row rows[r] with the sampler in slots[r]
        (int32 device tensors; None = r). Returns device tensors; asynchronous on the current stream."""
        if not logits.is_cuda or logits.dtype != torch.float32 or logits.dim() != 2 or logits.stride(1) != 1:
            raise ValueError("logits must be a 2-D fp32 CUDA tensor with contiguous rows")
        n_rows, V = logits.shape
        if V != self.vocab:
            raise ValueError(f"the samplers were built for a vocabulary of {self.vocab} and got {V} logits")
        B = int(rows.numel()) if rows is not None else (int(slots.numel()) if slots is not None else n_rows)
        dev = self.device
        if self._ws is None or self._ws.bytes < capi.lib().molla_sample_workspace_bytes(B, V, top_n):
            self._ws = Workspace(max(B, 1), V, top_n, dev)
        tokens = torch.empty(B, dtype=torch.int32, device=dev)
        status = torch.empty(B, dtype=torch.int32, device=dev)
        stopped = torch.empty(B, dtype=torch.uint8, device=dev)
        chosen = torch.empty(B, dtype=torch.float32, device=dev) if want_logprob else None
        top_ids = torch.empty((B, top_n), dtype=torch.int32, device=dev) if top_n else None
        top_lps = torch.empty((B, top_n), dtype=torch.float32, device=dev) if top_n else None
        b_ids, b_vals, b_off = self._bias_arrays()
        rc = capi.lib().molla_sample_decode_step(
            _ptr(logits), logits.stride(0), n_rows, V, _ptr(rows), _ptr(slots), B, self.n_slots, float(final_softcap),
            _ptr(self.temperature), _ptr(self.top_k), _ptr(self.top_p), _ptr(self.min_p), _ptr(self.typical_p),
            _ptr(self.repeat_penalty), _ptr(self.frequency_penalty), _ptr(self.presence_penalty),
            _ptr(self.seed), _ptr(self.drawn), _ptr(self.ring), self.ring_cap, _ptr(self.ring_head),
            _ptr(self.ring_filled), _ptr(self.ring_len), _ptr(self.stop_token), _ptr(b_ids), _ptr(b_vals), _ptr(b_off),
            top_n, _ptr(self._ws.buf), self._ws.bytes, _stream_ptr(dev), _ptr(tokens), _ptr(stopped), _ptr(chosen),
            _ptr(top_ids), _ptr(top_lps), _ptr(status))
        capi.check(rc)
        return dict(tokens=tokens, stopped=stopped, row_status=status, chosen_logprob=chosen, top_ids=top_ids,
                    top_logprobs=top_lps)
