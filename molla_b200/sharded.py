"""Row-sharded and vocab-sharded sampling over several GPUs of one node.

Row-sharded: rows are independent (per-sequence sampler state and a counter-based RNG,
src/molla/engine/sample.mojo:30-37,157-163), so every rank samples its own contiguous block
of rows with no collective (`row_range`).

Vocab-sharded (a tensor-parallel LM head): rank g holds columns [g*Vs, (g+1)*Vs) of every
row. Three library stages with two all-gathers between them (`sample_vocab_sharded`); the
collectives go through `torch.distributed` (NCCL over NVLink on GPUs), or through any
callable with the same contract, which is how one GPU stands in for several in the tests.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import capi
from .sampler import Workspace, _ptr, _stream_ptr


def row_range(rank: int, world: int, B: int) -> tuple[int, int]:
    """Contiguous rows [lo, hi) of rank `rank`; the first B % world ranks take one more."""
    base, extra = divmod(B, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def dist_all_gather(group=None):
    """An all-gather callable over a torch.distributed group: tensor -> [world, *tensor.shape]."""
    import torch.distributed as dist

    def gather(t: torch.Tensor) -> torch.Tensor:
        world = dist.get_world_size(group)
        out = torch.empty((world,) + tuple(t.shape), dtype=t.dtype, device=t.device)
        if dist.get_backend(group) == "nccl":
            dist.all_gather_into_tensor(out, t.contiguous(), group=group)
        else:  # gloo (CPU tests): the list form
            dist.all_gather(list(out.unbind(0)), t.contiguous(), group=group)
        return out

    return gather


class VocabShard:
    """One rank's part of a vocab-sharded sampling step."""

    def __init__(self, B: int, V_local: int, col0: int, V_global: int, rank: int, world: int, device,
                 list_cap: int | None = None):
        if world > 16:
            raise ValueError("at most 16 vocabulary shards")
        self.B, self.Vl, self.col0, self.Vg = B, V_local, col0, V_global
        # Before a row's largest logits have gone by, the running softmax sum is small and nearly every
        # logit can still move its last bit, so a shard's list can be as long as its slice: that is the
        # capacity that never overflows. A smaller one trades exchange volume for MOLLA_ROW_SHARD_OVERFLOW.
        if list_cap is None:
            list_cap = V_local
        self.rank, self.world, self.dev, self.cap = rank, world, torch.device(device), list_cap
        self.words = capi.lib().molla_sample_shard_summary_words()
        self.ws_local = Workspace(B, V_local, 0, self.dev)
        self.ws_global = Workspace(B, V_global, 0, self.dev)
        f32, i32, i64 = torch.float32, torch.int32, torch.int64
        self.summary = torch.empty((B, self.words), dtype=f32, device=self.dev)
        self.global4 = torch.empty((B, 4), dtype=f32, device=self.dev)
        self.lst = torch.empty((B, list_cap), dtype=i64, device=self.dev)
        self.count = torch.empty(B, dtype=i32, device=self.dev)
        self.tokens = torch.full((B,), -1, dtype=i32, device=self.dev)
        self.status = torch.zeros(B, dtype=i32, device=self.dev)

    def _row_args(self, p):
        g = p.get
        return [_ptr(g("temperature")), _ptr(g("top_k")), _ptr(g("top_p")), _ptr(g("min_p")), _ptr(g("typical_p")),
                _ptr(g("repeat_penalty")), _ptr(g("frequency_penalty")), _ptr(g("presence_penalty")),
                _ptr(g("window_on")), _ptr(g("hist")), _ptr(g("hist_off")), _ptr(g("bias_ids")),
                _ptr(g("bias_vals")), _ptr(g("bias_off"))]

    def stage_a(self, logits: torch.Tensor, p: dict) -> torch.Tensor:
        capi.check(capi.lib().molla_sample_shard_stage_a(
            _ptr(logits), logits.stride(0), self.B, self.Vl, self.col0, self.Vg, *self._row_args(p),
            _ptr(self.ws_local.buf), self.ws_local.bytes, _stream_ptr(self.dev), _ptr(self.summary)))
        return self.summary

    def merge(self, gathered: torch.Tensor, p: dict) -> torch.Tensor:
        g = p.get
        capi.check(capi.lib().molla_sample_shard_merge(
            self.B, self.Vg, self.world, self.rank, _ptr(g("temperature")), _ptr(g("top_k")),
            _ptr(gathered.contiguous()), _stream_ptr(self.dev), _ptr(self.global4), _ptr(self.tokens),
            _ptr(self.status)))
        return self.global4

    def stage_b(self, logits: torch.Tensor, p: dict):
        capi.check(capi.lib().molla_sample_shard_stage_b(
            _ptr(logits), logits.stride(0), self.B, self.Vl, self.col0, self.Vg, *self._row_args(p),
            _ptr(self.global4), self.cap, _ptr(self.ws_local.buf), self.ws_local.bytes, _stream_ptr(self.dev),
            _ptr(self.lst), _ptr(self.count)))
        return self.lst, self.count

    def stage_c(self, lists: torch.Tensor, counts: torch.Tensor, p: dict, diag: torch.Tensor | None = None):
        g = p.get
        capi.check(capi.lib().molla_sample_shard_stage_c(
            self.B, self.Vg, _ptr(g("temperature")), _ptr(g("top_k")), _ptr(g("top_p")), _ptr(g("min_p")),
            _ptr(g("typical_p")), _ptr(g("seed")), _ptr(g("drawn")), _ptr(self.global4), self.world, self.cap,
            _ptr(lists.contiguous()), _ptr(counts.contiguous()), _ptr(self.ws_global.buf), self.ws_global.bytes,
            _stream_ptr(self.dev), _ptr(self.tokens), _ptr(self.status), _ptr(diag)))
        return self.tokens, self.status


def sample_vocab_sharded(shard: VocabShard, logits: torch.Tensor, p: dict, all_gather, diag=None):
    """One sampling step on this rank's columns. `all_gather(t)` must return [world, *t.shape]
    with the shards in column order. Every rank ends with the same tokens."""
    gathered = all_gather(shard.stage_a(logits, p))
    shard.merge(gathered, p)
    lst, cnt = shard.stage_b(logits, p)
    return shard.stage_c(all_gather(lst), all_gather(cnt), p, diag)


def overflowed(counts: torch.Tensor, cap: int) -> torch.Tensor:
    """Rows whose list outgrew the exchange buffer on some shard: [world, B] gathered counts ->
    [B] bool. Every rank holds the same counts after the all-gather, so every rank comes to the
    same verdict about every row without talking again (stage c marks exactly these rows with
    MOLLA_ROW_SHARD_OVERFLOW and answers -1 for them)."""
    return ((counts < 0) | (counts > cap)).any(dim=0)


class NcclShardedSampler:
    """The vocab-sharded step through `molla_sample_sharded_step`: one C call per step that
    enqueues the stages and owns the all-gathers (NCCL, loaded by the library itself). The
    communicator is the library's own: rank 0 asks the library for an id, `share(id_bytes)` hands
    it to the other ranks (any broadcast of 128 bytes will do), every rank creates its
    communicator with its GPU current."""

    def __init__(self, B: int, V_local: int, col0: int, V_global: int, rank: int, world: int, device, share,
                 list_cap: int | None = None):
        self.B, self.Vl, self.col0, self.Vg, self.rank, self.world = B, V_local, col0, V_global, rank, world
        self.dev = torch.device(device)
        self.cap = V_local if list_cap is None else int(list_cap)
        L = capi.lib()
        ident = (C.c_uint8 * 128)()
        if rank == 0:
            self._check(L.molla_sample_nccl_unique_id(C.cast(ident, C.c_void_p)))
        ident = (C.c_uint8 * 128).from_buffer_copy(share(bytes(ident)))
        comm = C.c_void_p()
        with torch.cuda.device(self.dev):
            self._check(L.molla_sample_nccl_comm_create(C.cast(ident, C.c_void_p), rank, world, C.byref(comm)))
        self.comm = comm
        n = L.molla_sample_sharded_workspace_bytes(B, V_local, V_global, world, self.cap)
        if n < 0:
            self._check(int(n))
        self.ws = torch.empty(max(int(n), 256), dtype=torch.uint8, device=self.dev)
        self.tokens = torch.full((B,), -1, dtype=torch.int32, device=self.dev)
        self.status = torch.zeros(B, dtype=torch.int32, device=self.dev)
        self.wire = (C.c_int64 * 3)()

    @staticmethod
    def _check(rc: int) -> None:
        if rc != capi.OK:
            text = (capi.lib().molla_sample_sharded_last_error() or b"").decode("utf-8", "replace") or capi.last_error()
            raise capi.MollaSampleError(rc, text)

    def step(self, logits: torch.Tensor, p: dict, diag: torch.Tensor | None = None):
        g = p.get
        rc = capi.lib().molla_sample_sharded_step(
            self.comm, self.rank, self.world, _ptr(logits), logits.stride(0), self.B, self.Vl, self.col0, self.Vg,
            _ptr(g("temperature")), _ptr(g("top_k")), _ptr(g("top_p")), _ptr(g("min_p")), _ptr(g("typical_p")),
            _ptr(g("repeat_penalty")), _ptr(g("frequency_penalty")), _ptr(g("presence_penalty")), _ptr(g("window_on")),
            _ptr(g("hist")), _ptr(g("hist_off")), _ptr(g("bias_ids")), _ptr(g("bias_vals")), _ptr(g("bias_off")),
            _ptr(g("seed")), _ptr(g("drawn")), self.cap, _ptr(self.ws), self.ws.numel(), _stream_ptr(self.dev),
            _ptr(self.tokens), _ptr(self.status), _ptr(diag), C.cast(self.wire, C.c_void_p))
        self._check(rc)
        return self.tokens, self.status

    @property
    def wire_bytes(self) -> dict:
        return {"sent_per_rank": int(self.wire[0]), "received_per_rank": int(self.wire[1]),
                "list_entries_per_row": int(self.wire[2])}

    def close(self) -> None:
        if self.comm:
            capi.lib().molla_sample_nccl_comm_destroy(self.comm)
            self.comm = None


def share_over_torch_distributed(group=None):
    """A `share` callable for NcclShardedSampler: rank 0's bytes to everybody over torch.distributed."""
    import torch.distributed as dist

    def share(blob: bytes) -> bytes:
        box = [blob]
        dist.broadcast_object_list(box, src=0, group=group)
        return box[0]

    return share
