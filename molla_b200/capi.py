"""ctypes binding of libmolla_sample.so, the C ABI declared in include/molla_sample.h.

There is no fallback: if the shared library is missing or does not load, importing
callers get an error that says so. The library is built in-tree by
`molla_b200.build.build_library()`.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("MOLLA_SAMPLE_LIB", os.path.join(_HERE, "lib", "libmolla_sample.so"))

# status codes and row-status bits (mirrors of the header's #defines)
OK = 0
ERR_ARGUMENT, ERR_VOCAB, ERR_WORKSPACE, ERR_CONFIG = -1, -2, -3, -4
ERR_CUDA, ERR_DEVICE = 1, 2
NOALLOC_MAX_VOCAB = 262144
NOALLOC_MAX_ROWS = 4096
ROW_INVALID_CONFIG = 0x001
ROW_UNSUPPORTED = 0x002
ROW_TOPK_TIE = 0x004
ROW_TOPP_TIE = 0x008
ROW_CHOSEN_TIE = 0x010
ROW_LOAD_TIMEOUT = 0x020
ROW_SLOW_PATH = 0x040
ROW_DEGENERATE = 0x080
ROW_SHARD_OVERFLOW = 0x100
ROW_EMPTY = 0x200
ROW_TIE_BITS = ROW_TOPK_TIE | ROW_TOPP_TIE | ROW_CHOSEN_TIE
ROW_ERROR_BITS = ROW_INVALID_CONFIG | ROW_UNSUPPORTED | ROW_LOAD_TIMEOUT | ROW_DEGENERATE | ROW_SHARD_OVERFLOW | ROW_EMPTY

EXPORTS = (
    "molla_sample_abi_version", "molla_sample_last_error", "molla_sample_draw",
    "molla_sample_workspace_bytes", "molla_sample_batch", "molla_sample_batch_masked", "molla_sample_host_workspace_bytes",
    "molla_sample_batch_host", "molla_sample_batch_noalloc", "molla_sample_shard_summary_words",
    "molla_sample_shard_stage_a", "molla_sample_shard_merge", "molla_sample_shard_stage_b", "molla_sample_shard_stage_c", "molla_sample_penalised",
    "molla_sample_decode_step", "molla_sample_logprobs", "molla_sample_expf", "molla_sample_logf", "molla_sample_sync",
    "molla_sample_nccl_unique_id", "molla_sample_nccl_comm_create", "molla_sample_nccl_comm_destroy",
    "molla_sample_sharded_last_error", "molla_sample_sharded_workspace_bytes", "molla_sample_sharded_step",
)
TESTING_EXPORTS = ("molla_sample_debug_knobs", "molla_sample_debug_profile", "molla_sample_debug_topk")
TESTING_LIB_PATH = os.path.join(_HERE, "lib", "libmolla_sample_testing.so")


class MollaSampleError(RuntimeError):
    def __init__(self, status: int, text: str):
        super().__init__(f"molla_sample status {status}: {text}")
        self.status = status


_lib = None
_testing_lib = None


def lib():
    """The loaded library. Raises if it is not there: nothing else can do its work."""
    global _lib
    if _lib is None:
        _lib = _load(LIB_PATH, testing=False)
    return _lib


class testing_library:
    """`with capi.testing_library() as L:` routes every call of this package through
    libmolla_sample_testing.so (the same kernels built with their profiling stamps and experiment
    switches, see include/molla_sample_testing.h) and back to the production library afterwards."""

    def __enter__(self):
        global _lib, _testing_lib
        if _testing_lib is None:
            _testing_lib = _load(TESTING_LIB_PATH, testing=True)
        self._saved = _lib
        _lib = _testing_lib
        return _testing_lib

    def __exit__(self, *exc):
        global _lib
        _lib = self._saved
        return False


def _load(path, testing):
    if not os.path.exists(path):
        raise RuntimeError(
            f"{path} is missing: build it with `python -m molla_b200.build` "
            "(there is no CPU or PyTorch fallback for the sampling kernels)")
    L = C.CDLL(path)
    vp, i32, i64, u64, f32 = C.c_void_p, C.c_int32, C.c_int64, C.c_uint64, C.c_float
    L.molla_sample_abi_version.restype = i32
    L.molla_sample_abi_version.argtypes = []
    L.molla_sample_last_error.restype = C.c_char_p
    L.molla_sample_last_error.argtypes = []
    L.molla_sample_draw.restype = f32
    L.molla_sample_draw.argtypes = [u64, u64]
    L.molla_sample_workspace_bytes.restype = i64
    L.molla_sample_workspace_bytes.argtypes = [i32, i32, i32]
    L.molla_sample_batch.restype = i32
    L.molla_sample_batch.argtypes = [vp, i64, i32, i32] + [vp] * 16 + [i32, vp, i64, vp] + [vp] * 6
    L.molla_sample_batch_masked.restype = i32
    L.molla_sample_batch_masked.argtypes = [vp, i64] + L.molla_sample_batch.argtypes
    L.molla_sample_decode_step.restype = i32
    L.molla_sample_decode_step.argtypes = ([vp, i64, i32, i32, vp, vp, i32, i32, f32] + [vp] * 8 + [vp, vp, vp, i32, vp, vp, vp, vp]
                                           + [vp, vp, vp, i32, vp, i64, vp] + [vp] * 6)
    L.molla_sample_host_workspace_bytes.restype = i64
    L.molla_sample_host_workspace_bytes.argtypes = [i32, i32, i64, i64, i32]
    L.molla_sample_batch_host.restype = i32
    L.molla_sample_batch_host.argtypes = [vp, i64, i32, i32] + [vp] * 16 + [i32, vp, i64, vp] + [vp] * 5
    L.molla_sample_batch_noalloc.restype = i32
    L.molla_sample_batch_noalloc.argtypes = [vp, i64, i32, i32] + [vp] * 16 + [i32, vp] + [vp] * 5
    L.molla_sample_shard_summary_words.restype = i32
    L.molla_sample_shard_summary_words.argtypes = []
    L.molla_sample_shard_stage_a.restype = i32
    L.molla_sample_shard_stage_a.argtypes = [vp, i64, i32, i32, i32, i32] + [vp] * 14 + [vp, i64, vp, vp]
    L.molla_sample_shard_merge.restype = i32
    L.molla_sample_shard_merge.argtypes = [i32, i32, i32, i32, vp, vp, vp, vp, vp, vp, vp]
    L.molla_sample_shard_stage_b.restype = i32
    L.molla_sample_shard_stage_b.argtypes = [vp, i64, i32, i32, i32, i32] + [vp] * 14 + [vp, i32, vp, i64, vp, vp, vp]
    L.molla_sample_shard_stage_c.restype = i32
    L.molla_sample_shard_stage_c.argtypes = [i32, i32] + [vp] * 8 + [i32, i32, vp, vp, vp, i64, vp, vp, vp, vp]
    L.molla_sample_penalised.restype = i32
    L.molla_sample_penalised.argtypes = [vp, i64, i32, i32] + [vp] * 9 + [vp, i64, vp, vp]
    L.molla_sample_logprobs.restype = i32
    L.molla_sample_logprobs.argtypes = [vp, i64, i32, i32, vp, vp]
    L.molla_sample_expf.restype = i32
    L.molla_sample_expf.argtypes = [vp, i64, vp, vp]
    L.molla_sample_logf.restype = i32
    L.molla_sample_logf.argtypes = [vp, i64, vp, vp]
    L.molla_sample_sync.restype = i32
    L.molla_sample_sync.argtypes = [vp]
    L.molla_sample_nccl_unique_id.restype = i32
    L.molla_sample_nccl_unique_id.argtypes = [vp]
    L.molla_sample_nccl_comm_create.restype = i32
    L.molla_sample_nccl_comm_create.argtypes = [vp, i32, i32, C.POINTER(vp)]
    L.molla_sample_nccl_comm_destroy.restype = i32
    L.molla_sample_nccl_comm_destroy.argtypes = [vp]
    L.molla_sample_sharded_last_error.restype = C.c_char_p
    L.molla_sample_sharded_last_error.argtypes = []
    L.molla_sample_sharded_workspace_bytes.restype = i64
    L.molla_sample_sharded_workspace_bytes.argtypes = [i32, i32, i32, i32, i32]
    L.molla_sample_sharded_step.restype = i32
    L.molla_sample_sharded_step.argtypes = ([vp, i32, i32, vp, i64, i32, i32, i32, i32] + [vp] * 16
                                            + [i32, vp, i64, vp, vp, vp, vp, vp])
    if testing:
        L.molla_sample_debug_knobs.restype = None
        L.molla_sample_debug_knobs.argtypes = [i32]
        L.molla_sample_debug_profile.restype = None
        L.molla_sample_debug_profile.argtypes = [vp]
        L.molla_sample_debug_topk.restype = None
        L.molla_sample_debug_topk.argtypes = [vp, i32]
    return L


def last_error() -> str:
    return (lib().molla_sample_last_error() or b"").decode("utf-8", "replace")


def check(status: int) -> None:
    if status != OK:
        raise MollaSampleError(status, last_error())


def draw(seed: int, counter: int) -> float:
    m = (1 << 64) - 1
    return float(lib().molla_sample_draw(seed & m, counter & m))
