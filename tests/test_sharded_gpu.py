"""The vocab-sharded form on one GPU: the shards run one after another on the same device
and the two all-gathers are emulated by stacking their outputs. The result must be the
unsharded oracle's, bit for bit, like the single-GPU call's."""
import numpy as np
import pytest
import torch

from molla_b200 import capi, sampler as S, sharded, workloads as W

pytestmark = pytest.mark.gpu


def run_sharded(w, world, dev, list_cap=None, check_all_ranks=False):
    B, V = w["logits"].shape
    assert V % world == 0
    Vs = V // world
    p = S.upload_params(w, dev)
    full = torch.from_numpy(w["logits"]).to(dev)
    slices = [full[:, g * Vs:(g + 1) * Vs] for g in range(world)]  # row stride stays V
    shards = [sharded.VocabShard(B, Vs, g * Vs, V, g, world, dev, list_cap) for g in range(world)]
    summaries = torch.stack([sh.stage_a(sl, p).clone() for sh, sl in zip(shards, slices)])
    for sh in shards:
        sh.merge(summaries, p)
    outs = [sh.stage_b(sl, p) for sh, sl in zip(shards, slices)]
    lists = torch.stack([o[0] for o in outs])
    counts = torch.stack([o[1] for o in outs])
    diag = torch.zeros((B, 4), dtype=torch.float32, device=dev)
    ranks = range(world) if check_all_ranks else [0]
    res = []
    for g in ranks:
        tok, st = shards[g].stage_c(lists, counts, p, diag)
        torch.cuda.synchronize()
        res.append((tok.cpu().numpy().copy(), st.cpu().numpy().astype(np.uint32).copy()))
    for t, s in res[1:]:
        assert np.array_equal(t, res[0][0]) and np.array_equal(s, res[0][1])
    return res[0][0], res[0][1], diag.cpu().numpy(), counts.cpu().numpy()


def check(w, world, dev, oracle, **kw):
    kwargs = {k: w[k] for k in W.SAMPLER_KEYS}
    ref = oracle.pick_batch(w["logits"], **kwargs)
    tok, st, diag, counts = run_sharded(w, world, dev, **kw)
    assert not np.any(st & np.uint32(capi.ROW_ERROR_BITS)), np.unique(st)
    sampled = (w["temperature"] > 0) & (w["top_k"] != 1)
    assert np.array_equal(diag[sampled, 0].view(np.uint32), ref["z_sum"][sampled].view(np.uint32))
    tie = ((st & np.uint32(capi.ROW_TIE_BITS)) != 0) | ((ref["flags"] & 7) != 0)
    edge = (ref["flags"] & oracle.FLAG_CDF_EDGE) != 0
    bad = (tok != ref["tokens"]) & ~tie & ~edge
    assert not bad.any(), (np.nonzero(bad)[0][:8], tok[bad][:8], ref["tokens"][bad][:8])
    # and the same tokens as the unsharded call on one GPU
    one = S.sample_batch(torch.from_numpy(w["logits"]).to(dev), S.upload_params(w, dev))
    assert np.array_equal(tok[~tie], one["tokens"].cpu().numpy()[~tie])
    return counts


def test_config5_eight_shards(dev, lib, oracle):
    w = W.config5()  # all 128 rows of the configuration
    counts = check(w, 8, dev, oracle, check_all_ranks=True)
    assert counts.max() <= 18992 and counts.min() >= 0


def test_heterogeneous_rows_four_shards(dev, lib, oracle):
    w = W.config3(seed=77, B=48, V=151936)
    w["top_p"][5] = 1.0; w["top_k"][5] = 0; w["temperature"][5] = 0.9    # nothing sorts: vocabulary order
    w["top_p"][6] = 1.0; w["top_k"][6] = 30; w["temperature"][6] = 1.2   # top-k only
    check(w, 4, dev, oracle)


def test_small_vocabulary_two_shards(dev, lib, oracle):
    check(W.config3(seed=5, B=16, V=64, H=8), 2, dev, oracle)


def test_list_overflow_is_reported(dev, lib):
    w = W.config3(seed=9, B=8, V=32000)
    w["temperature"][:] = 1.4; w["top_k"][:] = 0; w["top_p"][:] = 0.9
    tok, st, _, counts = run_sharded(w, 2, dev, list_cap=256)
    assert (counts == -1).any()
    assert np.all((st & np.uint32(capi.ROW_SHARD_OVERFLOW)) != 0)
