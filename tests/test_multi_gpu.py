"""Two real GPUs, NCCL: the vocab-sharded form end to end under torch.distributed. Skipped
on boxes with fewer than two GPUs (the one-GPU emulation in test_sharded_gpu.py covers the
kernels; this covers the collectives)."""
import os
import sys

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    from molla_b200 import sampler as S, sharded, workloads as W
    w = W.config5(B=32)
    B, V = w["logits"].shape
    Vs = V // world
    local = torch.from_numpy(np.ascontiguousarray(w["logits"][:, rank * Vs:(rank + 1) * Vs])).to(dev)
    p = S.upload_params(w, dev)
    shard = sharded.VocabShard(B, Vs, rank * Vs, V, rank, world, dev)
    tok, st = sharded.sample_vocab_sharded(shard, local, p, sharded.dist_all_gather())
    torch.cuda.synchronize()
    np.save(os.path.join(out_dir, f"tok{rank}.npy"), tok.cpu().numpy())
    np.save(os.path.join(out_dir, f"st{rank}.npy"), st.cpu().numpy())
    dist.barrier()
    dist.destroy_process_group()


def test_vocab_sharded_over_nccl(tmp_path, oracle):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    world = 2
    mp.spawn(_worker, args=(world, 29600 + os.getpid() % 1000, str(tmp_path)), nprocs=world, join=True)
    from molla_b200 import capi, workloads as W
    w = W.config5(B=32)
    ref = oracle.pick_batch(w["logits"], **{k: w[k] for k in W.SAMPLER_KEYS})
    t0, t1 = np.load(tmp_path / "tok0.npy"), np.load(tmp_path / "tok1.npy")
    st = np.load(tmp_path / "st0.npy").astype(np.uint32)
    assert np.array_equal(t0, t1)
    assert not np.any(st & np.uint32(capi.ROW_ERROR_BITS))
    tie = ((st & np.uint32(capi.ROW_TIE_BITS)) != 0) | ((ref["flags"] & 7) != 0)
    assert np.array_equal(t0[~tie], ref["tokens"][~tie])


def _worker_c_abi(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)   # only to hand the id round
    from molla_b200 import sampler as S, sharded, workloads as W
    w = W.config5()   # all 128 rows of the configuration
    B, V = w["logits"].shape
    Vs = V // world
    local = torch.from_numpy(np.ascontiguousarray(w["logits"][:, rank * Vs:(rank + 1) * Vs])).to(dev)
    p = S.upload_params(w, dev)
    sh = sharded.NcclShardedSampler(B, Vs, rank * Vs, V, rank, world, dev, sharded.share_over_torch_distributed())
    diag = torch.zeros((B, 4), dtype=torch.float32, device=dev)
    for _ in range(2):   # the second step reuses the communicator and the workspace
        tok, st = sh.step(local, p, diag)
    torch.cuda.synchronize()
    np.save(os.path.join(out_dir, f"ctok{rank}.npy"), tok.cpu().numpy())
    np.save(os.path.join(out_dir, f"cst{rank}.npy"), st.cpu().numpy())
    np.save(os.path.join(out_dir, f"cdiag{rank}.npy"), diag.cpu().numpy())
    np.save(os.path.join(out_dir, f"cwire{rank}.npy"), np.array(list(sh.wire_bytes.values())))
    dist.barrier()
    sh.close()
    dist.destroy_process_group()


def test_sharded_step_through_the_c_abi_over_nccl(tmp_path, oracle):
    """`molla_sample_sharded_step`: the library's own communicator and all-gathers, config 5 at its
    full 128 rows over as many shards as the box has GPUs (2, 4 or 8)."""
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs two GPUs")
    world = 8 if n >= 8 else (4 if n >= 4 else 2)
    import torch.multiprocessing as mp
    mp.spawn(_worker_c_abi, args=(world, 29700 + os.getpid() % 1000, str(tmp_path)), nprocs=world, join=True)
    from molla_b200 import capi, workloads as W
    w = W.config5()
    ref = oracle.pick_batch(w["logits"], **{k: w[k] for k in W.SAMPLER_KEYS})
    toks = [np.load(tmp_path / f"ctok{r}.npy") for r in range(world)]
    st = np.load(tmp_path / "cst0.npy").astype(np.uint32)
    diag = np.load(tmp_path / "cdiag0.npy")
    for t in toks[1:]:
        assert np.array_equal(t, toks[0])
    assert not np.any(st & np.uint32(capi.ROW_ERROR_BITS))
    assert np.array_equal(diag[:, 0].view(np.uint32), ref["z_sum"].view(np.uint32))   # the softmax denominators, bit for bit
    tie = ((st & np.uint32(capi.ROW_TIE_BITS)) != 0) | ((ref["flags"] & 7) != 0)
    assert np.array_equal(toks[0][~tie], ref["tokens"][~tie])
    print("wire bytes per rank (sent, received, list entries per row):", np.load(tmp_path / "cwire0.npy"))
