"""The sampling entry point for callers that cannot allocate device memory.

Some callers sample from inside a loop whose device memory was divided up once and for
all (a fixed arena, another runtime's allocator, a region the device heap must not be
touched in), so they cannot provide the workspace `molla_sample_batch` asks for.
`molla_sample_batch_noalloc` uses a fixed array inside the library instead. This test
calls it through the C ABI twice in a row and checks each result against the ordinary
entry point: bit-identical tokens, status words and logprobs (integer outputs and the
same arithmetic, so no tolerance is needed). The file sorts last on purpose, so a run
that stops at the first failure has already run everything else.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from molla_b200 import capi, sampler as S, workloads as W

pytestmark = pytest.mark.gpu


def _ptr(t):
    return None if t is None else C.c_void_p(t.data_ptr())


def noalloc(logits, p, top_n):
    B, V = logits.shape
    dev = logits.device
    tokens = torch.full((B,), -7, dtype=torch.int32, device=dev)
    status = torch.full((B,), -7, dtype=torch.int32, device=dev)
    chosen = torch.zeros(B, dtype=torch.float32, device=dev)
    ids = torch.zeros((B, top_n), dtype=torch.int32, device=dev)
    lps = torch.zeros((B, top_n), dtype=torch.float32, device=dev)
    g = p.get
    rc = capi.lib().molla_sample_batch_noalloc(
        _ptr(logits), logits.stride(0), B, V,
        _ptr(g("temperature")), _ptr(g("top_k")), _ptr(g("top_p")), _ptr(g("min_p")), _ptr(g("typical_p")),
        _ptr(g("repeat_penalty")), _ptr(g("frequency_penalty")), _ptr(g("presence_penalty")),
        _ptr(g("window_on")), _ptr(g("seed")), _ptr(g("drawn")), _ptr(g("hist")), _ptr(g("hist_off")),
        _ptr(g("bias_ids")), _ptr(g("bias_vals")), _ptr(g("bias_off")), top_n,
        C.c_void_p(torch.cuda.current_stream(dev).cuda_stream),
        _ptr(tokens), _ptr(chosen), _ptr(ids), _ptr(lps), _ptr(status))
    capi.check(rc)
    torch.cuda.synchronize()
    return tokens.cpu().numpy(), status.cpu().numpy(), chosen.cpu().numpy(), ids.cpu().numpy(), lps.cpu().numpy()


def test_noalloc_matches_the_ordinary_entry_point_twice(dev, lib):
    top_n = 3
    # two different workloads back to back: the second call finds the first one's leftovers
    # in the built-in scratch (more rows than the scratch has room for thread blocks)
    for seed, B, V in ((41, 40, 151936), (42, 24, 30001)):
        w = W.config3(seed=seed, B=B, V=V, H=64)
        logits = torch.from_numpy(w["logits"]).to(dev)
        p = S.upload_params(w, dev)
        ref = S.sample_batch(logits, p, top_n=top_n, want_logprob=True)
        torch.cuda.synchronize()
        tok, st, ch, ids, lps = noalloc(logits, p, top_n)
        assert np.array_equal(tok, ref["tokens"].cpu().numpy())
        # the status words agree except for the informational bit that says a sequential fallback
        # ran (the two entry points do not run the same kernel)
        info = np.int32(capi.ROW_SLOW_PATH)
        assert np.array_equal(st & ~info, ref["row_status"].cpu().numpy() & ~info)
        assert np.array_equal(ch, ref["chosen_logprob"].cpu().numpy())
        assert np.array_equal(ids, ref["top_ids"].cpu().numpy())
        assert np.array_equal(lps, ref["top_logprobs"].cpu().numpy())
        assert np.all(tok >= 0)


def test_noalloc_refuses_sizes_beyond_its_scratch(dev, lib):
    V = capi.NOALLOC_MAX_VOCAB + 4
    logits = torch.zeros((1, V), dtype=torch.float32, device=dev)
    tokens = torch.zeros(1, dtype=torch.int32, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    null = C.c_void_p(None)
    args = [_ptr(logits), V, 1, V] + [null] * 16 + [0, null, _ptr(tokens), null, null, null, _ptr(status)]
    assert capi.lib().molla_sample_batch_noalloc(*args) == capi.ERR_WORKSPACE
    assert "MOLLA_NOALLOC_MAX_VOCAB" in capi.last_error()
