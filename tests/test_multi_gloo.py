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
