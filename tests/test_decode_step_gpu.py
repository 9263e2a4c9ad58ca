"""The decode-step form of the sampler (`molla_sample_decode_step`): logit rows picked by
`rows[]`, settings and state per sampler slot kept on the device, the final-logit softcap
fused into the read. Checked against oracle-backed samplers that keep their state on the host
the way the reference's `Sampler` does (src/molla/engine/sample.mojo:157-363) and, for the
softcap, against the oracle's restatement of the reference's device kernel
(src/molla/nn/gpu_ops.mojo:302-317, :607-623) applied to the block beforehand."""
import numpy as np
import pytest
import torch

from helpers import OracleSampler
from molla_b200 import capi, sampler as S

pytestmark = pytest.mark.gpu

CONFIGS = [
    dict(),                                                                    # greedy, window of 64 cut to the capacity
    dict(frequency_penalty=0.4, presence_penalty=0.2, repeat_last_n=8),        # greedy with penalties
    dict(temperature=0.8, top_k=40, top_p=0.9, repeat_penalty=1.2, repeat_last_n=16, seed=5),
    dict(temperature=1.0, top_p=0.95, seed=6, repeat_last_n=0),                # no window at all
    dict(temperature=1.3, seed=7, repeat_last_n=4, frequency_penalty=0.1),     # nothing sorted
    dict(temperature=0.7, top_k=20, min_p=0.05, seed=8, repeat_last_n=16, presence_penalty=0.5),
    dict(temperature=0.9, top_k=12, typical_p=0.8, seed=9, repeat_last_n=8),
    dict(temperature=1.1, top_k=1, seed=10, repeat_last_n=16, repeat_penalty=1.3),
    dict(temperature=0.5, top_p=0.5, seed=11, repeat_last_n=16),
    dict(temperature=2.0, top_k=300, top_p=0.99, seed=12, repeat_last_n=16, repeat_penalty=1.1),
]


def make(dev, oracle, V, ring_cap):
    ds = S.DeviceSamplers(len(CONFIGS), V, ring_cap=ring_cap, device=dev)
    host = []
    for slot, kw in enumerate(CONFIGS):
        kw = dict(kw)
        kw["repeat_last_n"] = min(kw.get("repeat_last_n", 64), ring_cap)
        bias = [(3, 2.5), (3, 0.5), (V - 1, -4.0)] if slot in (2, 5) else []
        ds.assign(slot, S.SamplerConfig(**kw), stop_token=7 if slot % 2 == 0 else -1, bias=bias)
        o = OracleSampler(oracle, V, **kw)
        for t, a in bias:
            o.bias(t, a)
        host.append(o)
    return ds, host


@pytest.mark.parametrize("softcap", [0.0, 30.0])
def test_decode_steps_match_host_kept_samplers(dev, lib, oracle, softcap):
    V, ring_cap, n_block = 3000, 16, 14
    ds, host = make(dev, oracle, V, ring_cap)
    rng = np.random.default_rng(77)
    for step in range(9):
        block = (3.0 * rng.standard_normal((n_block, V))).astype(np.float32)
        block[:, 7] += 4.0  # the stop token turns up now and then
        active = rng.permutation(len(CONFIGS))[: 6 + step % 4]
        rows = rng.permutation(n_block)[: len(active)]
        got = ds.step(torch.from_numpy(block).to(dev), torch.tensor(rows, dtype=torch.int32, device=dev),
                      torch.tensor(active, dtype=torch.int32, device=dev), final_softcap=softcap, want_logprob=True)
        torch.cuda.synchronize()
        st = got["row_status"].cpu().numpy()
        assert not np.any(st & np.uint32(capi.ROW_ERROR_BITS)), st
        seen = oracle.softcap(block, softcap) if softcap > 0 else block
        tok = got["tokens"].cpu().numpy()
        stopped = got["stopped"].cpu().numpy()
        lp = oracle.logprobs_batch(seen[rows], tokens=tok, top_n=0)
        assert np.max(np.abs(got["chosen_logprob"].cpu().numpy() - lp["chosen_logprob"])) <= 1e-5
        for i, slot in enumerate(active):
            want = host[slot].pick(seen[rows[i]])
            tie = st[i] & np.uint32(capi.ROW_TIE_BITS)
            if not tie:
                assert tok[i] == want, (step, slot, tok[i], want)
            elif tok[i] != want and host[slot].recent:  # keep the two histories the same past an order-dependent pick
                h = host[slot]
                h.recent[(h.head - 1) % len(h.recent)] = int(tok[i])
            assert stopped[i] == (1 if (slot % 2 == 0 and tok[i] == 7) else 0)
        # the state the kernel left is the state the host samplers are in
        drawn = ds.drawn.cpu().numpy()
        head, filled, ring = ds.ring_head.cpu().numpy(), ds.ring_filled.cpu().numpy(), ds.ring.cpu().numpy()
        for slot, h in enumerate(host):
            assert drawn[slot] == h.drawn
            assert filled[slot] == h.filled and (head[slot] == h.head or not h.recent)
            assert ring[slot, : h.filled].tolist() == h.recent[: h.filled]


def test_softcap_alone_is_bit_identical_to_the_oracle(dev, lib, oracle):
    """Penalised-value dump of a capped row = oracle softcap of the row (no penalties, no bias)."""
    V = 5000
    rng = np.random.default_rng(3)
    block = (40.0 * rng.standard_normal((4, V))).astype(np.float32)
    ds = S.DeviceSamplers(4, V, ring_cap=8, device=dev)
    for slot in range(4):
        ds.assign(slot, S.SamplerConfig(repeat_last_n=8))  # greedy
    got = ds.step(torch.from_numpy(block).to(dev), None, None, final_softcap=50.0, want_logprob=True)
    capped = oracle.softcap(block, 50.0)
    assert got["tokens"].cpu().numpy().tolist() == [int(np.argmax(r)) for r in capped]
    lp = oracle.logprobs_batch(capped, tokens=got["tokens"].cpu().numpy(), top_n=0)
    assert np.max(np.abs(got["chosen_logprob"].cpu().numpy() - lp["chosen_logprob"])) <= 1e-5
    assert np.all(np.abs(capped) <= 50.0)


def test_bad_arguments_are_refused_before_any_launch(dev, lib):
    ds = S.DeviceSamplers(2, 100, ring_cap=8, device=dev)
    ds.assign(0, S.SamplerConfig(repeat_last_n=8))
    ds.assign(1, S.SamplerConfig(repeat_last_n=0))
    with pytest.raises(ValueError):
        ds.assign(0, S.SamplerConfig(repeat_last_n=9))
    with pytest.raises(ValueError):
        ds.assign(5, S.SamplerConfig(repeat_last_n=8))
    with pytest.raises(ValueError):
        ds.step(torch.zeros((2, 99), device=dev), None, None)
    with pytest.raises(capi.MollaSampleError):
        ds.step(torch.zeros((2, 100), device=dev), None, None, final_softcap=-1.0)


def test_stale_row_and_slot_indices_touch_nothing(dev, lib):
    """`pick` refuses a row outside the block (sample.mojo:316-322). The device form reports such a
    row (and a slot outside the samplers) in its status word and reads and writes nothing of it.
    The tensors here are larger than the sizes declared to the call, so that a missing check would
    land in owned memory rather than fault."""
    V, declared_rows, declared_slots = 1000, 4, 3
    ds = S.DeviceSamplers(8, V, ring_cap=8, device=dev)          # 8 slots allocated, 3 declared
    for slot in range(8):
        ds.assign(slot, S.SamplerConfig(temperature=0.8, top_k=10, seed=slot, repeat_last_n=8))
    ds.n_slots = declared_slots
    block = torch.randn((8, V), device=dev)                      # 8 rows allocated, 4 declared
    rows = torch.tensor([0, 5, 2, -1, 3], dtype=torch.int32, device=dev)
    slots = torch.tensor([0, 1, 6, 2, 2], dtype=torch.int32, device=dev)
    before = {k: getattr(ds, k).clone() for k in ("drawn", "ring", "ring_head", "ring_filled")}
    got = ds.step(block[:declared_rows], rows, slots, want_logprob=True, top_n=3)
    torch.cuda.synchronize()
    st = got["row_status"].cpu().numpy().astype(np.uint32)
    tok = got["tokens"].cpu().numpy()
    for i in (1, 2, 3):   # row 5 of 4, slot 6 of 3, row -1
        assert st[i] & capi.ROW_INVALID_CONFIG and tok[i] == -1, (i, st[i], tok[i])
    assert st[0] == 0 and tok[0] >= 0 and (st[4] & capi.ROW_ERROR_BITS) == 0 and tok[4] >= 0
    drawn = ds.drawn.cpu().numpy()
    assert drawn[0] == 1 and drawn[2] == 1 and drawn[1] == 0 and drawn[6] == 0
    for k in ("ring", "ring_head", "ring_filled"):
        assert torch.equal(getattr(ds, k)[[1, 6]], before[k][[1, 6]]), k
    assert np.all(got["top_ids"].cpu().numpy()[[1, 3]] == -1)


def test_a_wait_that_ran_out_fails_the_row_and_keeps_its_state(dev, lib):
    """The bounded wait on a row's load reports in one warp only. The testing build can pretend
    that it ran out (nothing is withheld, nothing is left waiting): every such row must come back
    with MOLLA_ROW_LOAD_TIMEOUT and token -1, and the sampler in its slot must be as it was."""
    V = 20000
    ds = S.DeviceSamplers(4, V, ring_cap=8, device=dev)
    for slot in range(4):
        ds.assign(slot, S.SamplerConfig(temperature=0.0 if slot == 0 else 0.9, top_k=[0, 1, 20, 0][slot],
                                        top_p=0.9, seed=slot, repeat_last_n=8))
    block = torch.randn((4, V), device=dev)
    before = {k: getattr(ds, k).clone() for k in ("drawn", "ring", "ring_head", "ring_filled")}
    with capi.testing_library() as T:
        T.molla_sample_debug_knobs(16)
        try:
            got = ds.step(block, None, None)
            torch.cuda.synchronize()
        finally:
            T.molla_sample_debug_knobs(0)
    st = got["row_status"].cpu().numpy().astype(np.uint32)
    assert np.all(st & capi.ROW_LOAD_TIMEOUT), st
    assert np.all(got["tokens"].cpu().numpy() == -1)
    for k, v in before.items():
        assert torch.equal(getattr(ds, k), v), k
    # and the same samplers work on the next call
    got = ds.step(block, None, None)
    torch.cuda.synchronize()
    assert not np.any(got["row_status"].cpu().numpy().astype(np.uint32) & capi.ROW_ERROR_BITS)
    assert np.all(ds.drawn.cpu().numpy() == 1)
