"""ctypes binding of the CPU oracle. TEST INFRASTRUCTURE, NOT PRODUCT CODE.

Only the tests, the smoke test and the CPU-baseline leg of the benchmark import
this module; the shipped package never does. The library it loads is built from
`molla_oracle.c` by the Makefile beside it.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "_build", "libmolla_oracle.so")

FLAG_TOPK_TIE = 1
FLAG_TOPP_TIE = 2
FLAG_CHOSEN_TIE = 4
FLAG_CDF_EDGE = 8
FLAG_KEPT_TIE = 16


def build(force: bool = False) -> str:
    """Compile the oracle if its library is missing or older than its source."""
    src = os.path.join(_HERE, "molla_oracle.c")
    stale = (not os.path.exists(_SO)) or (
        os.path.exists(src) and os.path.getmtime(src) > os.path.getmtime(_SO)
    )
    if force or stale:
        subprocess.check_call(["make", "-C", _HERE, "-B" if force else "-s"])
    return _SO


_lib = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_SO):
            build()
        L = C.CDLL(_SO)
        L.molla_oracle_mix.restype = C.c_uint64
        L.molla_oracle_mix.argtypes = [C.c_uint64]
        L.molla_oracle_draw.restype = C.c_float
        L.molla_oracle_draw.argtypes = [C.c_uint64, C.c_uint64]
        L.molla_oracle_expf.restype = C.c_float
        L.molla_oracle_expf.argtypes = [C.c_float]
        L.molla_oracle_logf_array.restype = None
        L.molla_oracle_logf_array.argtypes = [C.c_void_p, C.c_int64, C.c_void_p]
        L.molla_oracle_softcap.restype = None
        L.molla_oracle_softcap.argtypes = [C.c_void_p, C.c_int64, C.c_float, C.c_void_p]
        L.molla_oracle_argmax.restype = C.c_int64
        L.molla_oracle_argmax.argtypes = [C.c_void_p, C.c_int64, C.c_int64]
        L.molla_oracle_logprobs.restype = None
        L.molla_oracle_logprobs.argtypes = [C.c_void_p, C.c_int64, C.c_void_p, C.c_int]
        L.molla_oracle_pick_batch.restype = C.c_int
        L.molla_oracle_logprobs_batch.restype = C.c_int
        L.molla_oracle_max_threads.restype = C.c_int
        _lib = L
    return _lib


def draw(seed: int, counter: int) -> float:
    return float(lib().molla_oracle_draw(C.c_uint64(seed & (2**64 - 1)), C.c_uint64(counter & (2**64 - 1))))


def mix(v: int) -> int:
    return int(lib().molla_oracle_mix(C.c_uint64(v & (2**64 - 1))))


def expf(x) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32).ravel()
    out = np.empty_like(x)
    f = lib().molla_oracle_expf
    for i in range(x.size):
        out[i] = f(C.c_float(float(x[i])))
    return out


def logf(x) -> np.ndarray:
    """The pinned fp32 logarithm of the typical-p filter, elementwise."""
    x = np.ascontiguousarray(x, dtype=np.float32).ravel()
    out = np.empty_like(x)
    lib().molla_oracle_logf_array(x.ctypes.data_as(C.c_void_p), x.size, out.ctypes.data_as(C.c_void_p))
    return out


def softcap(x, cap: float) -> np.ndarray:
    """cap * tanh(x / cap) as the reference's device kernel evaluates it, same shape as x."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty_like(x)
    lib().molla_oracle_softcap(x.ctypes.data_as(C.c_void_p), x.size, C.c_float(cap), out.ctypes.data_as(C.c_void_p))
    return out


def argmax(x, at: int = 0, n: int | None = None) -> int:
    x = np.ascontiguousarray(x, dtype=np.float32)
    if n is None:
        n = x.size - at
    return int(lib().molla_oracle_argmax(x.ctypes.data, at, n))


def logprobs(z, exp_mode: int = 0) -> np.ndarray:
    z = np.ascontiguousarray(z, dtype=np.float32).ravel()
    out = np.empty_like(z)
    lib().molla_oracle_logprobs(z.ctypes.data, z.size, out.ctypes.data, exp_mode)
    return out


def _p(a):
    return None if a is None else C.c_void_p(a.ctypes.data)


def _per_row(v, B, dtype, default):
    if v is None:
        return np.full(B, default, dtype=dtype)
    a = np.asarray(v, dtype=dtype)
    if a.ndim == 0:
        a = np.full(B, a, dtype=dtype)
    assert a.shape == (B,)
    return np.ascontiguousarray(a)


def pick_batch(
    logits,
    temperature=None,
    top_k=None,
    top_p=None,
    min_p=None,
    typical_p=None,
    repeat_penalty=None,
    frequency_penalty=None,
    presence_penalty=None,
    seed=None,
    drawn=None,
    hist=None,
    hist_off=None,
    window_on=None,
    bias_ids=None,
    bias_vals=None,
    bias_off=None,
    exp_mode: int = 0,
    faithful_cost: bool = False,
    nthreads: int = 0,
    want_penalised: bool = False,
    kept_ids_cap: int = 0,
    mask=None,
):
    """Sample every row of `logits` ([B, V] fp32) and return a dict of results."""
    logits = np.ascontiguousarray(logits, dtype=np.float32)
    if logits.ndim == 1:
        logits = logits[None, :]
    B, V = logits.shape
    if nthreads <= 0:
        nthreads = os.cpu_count() or 1
    temperature = _per_row(temperature, B, np.float32, 0.0)
    top_k = _per_row(top_k, B, np.int32, 0)
    top_p = _per_row(top_p, B, np.float32, 1.0)
    min_p = _per_row(min_p, B, np.float32, 0.0)
    typical_p = _per_row(typical_p, B, np.float32, 1.0)
    repeat_penalty = _per_row(repeat_penalty, B, np.float32, 1.0)
    frequency_penalty = _per_row(frequency_penalty, B, np.float32, 0.0)
    presence_penalty = _per_row(presence_penalty, B, np.float32, 0.0)
    seed = _per_row(seed, B, np.uint64, 0)
    drawn = _per_row(drawn, B, np.uint64, 0)
    if hist is not None:
        hist = np.ascontiguousarray(hist, dtype=np.int64)
        hist_off = np.ascontiguousarray(hist_off, dtype=np.int32)
        assert hist_off.shape == (B + 1,)
    if window_on is None:
        window_on = np.ones(B, dtype=np.uint8)
    window_on = _per_row(window_on, B, np.uint8, 1)
    if bias_ids is not None:
        bias_ids = np.ascontiguousarray(bias_ids, dtype=np.int64)
        bias_vals = np.ascontiguousarray(bias_vals, dtype=np.float32)
        bias_off = np.ascontiguousarray(bias_off, dtype=np.int32)
    tokens = np.empty(B, dtype=np.int32)
    penalised = np.empty((B, V), dtype=np.float32) if want_penalised else None
    z_sum = np.zeros(B, dtype=np.float32)
    keep_sum = np.zeros(B, dtype=np.float32)
    target = np.zeros(B, dtype=np.float32)
    chosen_p = np.zeros(B, dtype=np.float32)
    kept_topk = np.zeros(B, dtype=np.int32)
    kept_final = np.zeros(B, dtype=np.int32)
    flags = np.zeros(B, dtype=np.uint32)
    kept_ids = np.full((B, kept_ids_cap), -1, dtype=np.int32) if kept_ids_cap > 0 else None
    if mask is not None:
        mask = np.ascontiguousarray(mask, dtype=np.uint32)
        assert mask.shape == (B, (V + 31) // 32)
        want_penalised, penalised = False, None
    rc = lib().molla_oracle_pick_batch_masked(
        _p(mask), C.c_int64(0 if mask is None else mask.shape[1]),
        _p(logits), C.c_int64(V), C.c_int32(B), C.c_int32(V),
        _p(temperature), _p(top_k), _p(top_p), _p(min_p), _p(typical_p),
        _p(repeat_penalty), _p(frequency_penalty), _p(presence_penalty), _p(window_on),
        _p(seed), _p(drawn), _p(hist), _p(hist_off), _p(bias_ids), _p(bias_vals), _p(bias_off),
        C.c_int32(exp_mode), C.c_int32(1 if faithful_cost else 0), C.c_int32(nthreads),
        _p(tokens), _p(penalised), _p(z_sum), _p(keep_sum), _p(target), _p(chosen_p),
        _p(kept_topk), _p(kept_final), _p(flags), _p(kept_ids), C.c_int32(kept_ids_cap),
    )
    if rc != 0:
        raise ValueError("oracle refused its arguments")
    return dict(
        tokens=tokens, penalised=penalised, z_sum=z_sum, keep_sum=keep_sum, target=target,
        chosen_p=chosen_p, kept_topk=kept_topk, kept_final=kept_final, flags=flags,
        kept_ids=kept_ids,
    )


def logprobs_batch(logits, tokens=None, top_n: int = 0, exp_mode: int = 0, nthreads: int = 0):
    logits = np.ascontiguousarray(logits, dtype=np.float32)
    if logits.ndim == 1:
        logits = logits[None, :]
    B, V = logits.shape
    if nthreads <= 0:
        nthreads = os.cpu_count() or 1
    chosen = np.zeros(B, dtype=np.float32) if tokens is not None else None
    if tokens is not None:
        tokens = np.ascontiguousarray(tokens, dtype=np.int32)
    ids = np.zeros((B, top_n), dtype=np.int32) if top_n > 0 else None
    lps = np.zeros((B, top_n), dtype=np.float32) if top_n > 0 else None
    rc = lib().molla_oracle_logprobs_batch(
        _p(logits), C.c_int64(V), C.c_int32(B), C.c_int32(V), _p(tokens), C.c_int32(top_n),
        C.c_int32(exp_mode), C.c_int32(nthreads), _p(chosen), _p(ids), _p(lps),
    )
    if rc != 0:
        raise ValueError("oracle refused its arguments")
    return dict(chosen_logprob=chosen, top_ids=ids, top_logprobs=lps)


def max_threads() -> int:
    return int(lib().molla_oracle_max_threads())
