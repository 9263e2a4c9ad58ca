"""The multi-rank host logic on CPU: two gloo ranks. Row sharding (each rank takes a block of
rows, no data-path collective, tokens gathered on the host) and the all-gather layout the
vocab-sharded form relies on. The sampling itself is done by the CPU checker here: the
kernels need a GPU and are covered by the gpu-marked tests."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from molla_b200 import sharded, workloads as W
    from oracle import pyoracle as O
    w = W.config3(seed=123, B=13, V=3000, H=16)
    lo, hi = sharded.row_range(rank, world, w["B"])
    mine = W.slice_rows(w, lo, hi)
    kw = {k: mine[k] for k in W.SAMPLER_KEYS}
    tok = O.pick_batch(mine["logits"], **kw, nthreads=1)["tokens"]
    # host-side gather of the ragged token blocks
    sizes = [sharded.row_range(r, world, w["B"]) for r in range(world)]
    width = max(h - l for l, h in sizes)
    pad = torch.full((width,), -1, dtype=torch.int32)
    pad[: hi - lo] = torch.from_numpy(tok)
    got = sharded.dist_all_gather()(pad)
    assert got.shape == (world, width)
    full = np.concatenate([got[r, : h - l].numpy() for r, (l, h) in enumerate(sizes)])
    # the all-gather keeps rank order on every leading axis (what stage 3 of the sharded form indexes)
    tag = torch.full((2, 3), float(rank))
    g = sharded.dist_all_gather()(tag)
    assert g.shape == (world, 2, 3) and all(float(g[r, 0, 0]) == r for r in range(world))
    if rank == 0:
        np.save(os.path.join(out_dir, "tokens.npy"), full)
    dist.barrier()
    dist.destroy_process_group()


def test_row_ranges_partition_the_batch():
    from molla_b200.sharded import row_range
    for B in (0, 1, 7, 256, 1000):
        for world in (1, 2, 3, 8):
            spans = [row_range(r, world, B) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == B
            assert all(spans[i][1] == spans[i + 1][0] for i in range(world - 1))
            sizes = [h - l for l, h in spans]
            assert max(sizes) - min(sizes) <= 1


def test_two_ranks_row_sharded_equals_one(tmp_path):
    world, port = 2, 29500 + os.getpid() % 2000
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    sys.path.insert(0, ROOT)
    from molla_b200 import workloads as W
    from oracle import pyoracle as O
    w = W.config3(seed=123, B=13, V=3000, H=16)
    kw = {k: w[k] for k in W.SAMPLER_KEYS}
    ref = O.pick_batch(w["logits"], **kw)["tokens"]
    assert np.array_equal(np.load(tmp_path / "tokens.npy"), ref)


# ---- what the ranks of the vocab-sharded form do when one of them reports trouble ---------------

class _FakeShard:
    """The stages of a shard with the kernels replaced by stand-ins that produce the payloads'
    shapes (the kernels need a GPU): enough to drive `sample_vocab_sharded` on CPU ranks."""

    def __init__(self, rank, world, B, cap, bad_row=None):
        self.rank, self.world, self.B, self.cap, self.bad_row = rank, world, B, cap, bad_row

    def stage_a(self, logits, p):
        return torch.full((self.B, 4), float(self.rank))

    def merge(self, gathered, p):
        assert gathered.shape == (self.world, self.B, 4)

    def stage_b(self, logits, p):
        lst = torch.full((self.B, self.cap), self.rank, dtype=torch.int64)
        cnt = torch.full((self.B,), 2, dtype=torch.int32)
        if self.bad_row is not None:
            cnt[self.bad_row] = -1     # this shard's list outgrew the exchange buffer
        return lst, cnt

    def stage_c(self, lists, counts, p, diag):
        from molla_b200 import capi, sharded
        over = sharded.overflowed(counts, self.cap)
        status = torch.where(over, torch.tensor(capi.ROW_SHARD_OVERFLOW), torch.tensor(0)).to(torch.int32)
        tokens = torch.where(over, torch.tensor(-1), lists[:, :, 0].sum(0).to(torch.int64)).to(torch.int32)
        return tokens, status


def _worker_overflow(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from molla_b200 import sharded
    shard = _FakeShard(rank, world, B=6, cap=4, bad_row=3 if rank == 1 else None)
    tok, st = sharded.sample_vocab_sharded(shard, None, {}, sharded.dist_all_gather())
    np.save(os.path.join(out_dir, f"tok{rank}.npy"), tok.numpy())
    np.save(os.path.join(out_dir, f"st{rank}.npy"), st.numpy())
    dist.barrier()
    dist.destroy_process_group()


def test_an_overflow_on_one_shard_is_the_same_verdict_on_every_rank(tmp_path):
    """Rank 1 reports a list that did not fit. After the all-gather of the counts every rank holds
    the same counts, so every rank fails the same row (and only that row) without another exchange."""
    from molla_b200 import capi
    world, port = 2, 31500 + os.getpid() % 2000
    mp.spawn(_worker_overflow, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    t0, t1 = np.load(tmp_path / "tok0.npy"), np.load(tmp_path / "tok1.npy")
    s0, s1 = np.load(tmp_path / "st0.npy"), np.load(tmp_path / "st1.npy")
    assert np.array_equal(t0, t1) and np.array_equal(s0, s1)
    assert s0[3] == capi.ROW_SHARD_OVERFLOW and t0[3] == -1
    others = np.arange(6) != 3
    assert np.all(s0[others] == 0) and np.all(t0[others] == 1)   # ranks 0 + 1: the stand-in's "token"


def _worker_lost_peer(rank, world, port, out_dir):
    import datetime
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=8))
    from molla_b200 import sharded
    gather = sharded.dist_all_gather()
    gather(torch.zeros(4))               # the first exchange of a step goes through
    if rank == 1:
        os._exit(0)                      # the rank is gone between two exchanges (on the host: no GPU involved)
    try:
        gather(torch.zeros(4))           # the survivor's next exchange must fail, not hang
        outcome = "completed"
    except Exception as e:               # gloo: connection closed by peer / timed out
        outcome = "error: " + type(e).__name__
    open(os.path.join(out_dir, "outcome.txt"), "w").write(outcome)
    os._exit(0)


def test_a_lost_rank_ends_the_next_exchange_with_an_error(tmp_path):
    world, port = 2, 33500 + os.getpid() % 2000
    mp.spawn(_worker_lost_peer, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    assert open(tmp_path / "outcome.txt").read().startswith("error")
