"""The C ABI without a GPU: the library loads, exports every function the header
declares, and refuses bad arguments before it touches the device."""
import ctypes as C
import os
import re

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions(header="molla_sample.h"):
    text = open(os.path.join(ROOT, "include", header)).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(molla_sample_\w+)\s*\(", text)))


def test_every_declared_symbol_is_exported(lib):
    from molla_b200 import capi
    names = declared_functions()
    assert len(names) >= 10
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in the header but not exported"
    assert set(capi.EXPORTS) <= set(names)
    assert lib.molla_sample_abi_version() == 1


def test_testing_aids_live_in_the_testing_library_only(lib):
    from molla_b200 import capi
    names = declared_functions("molla_sample_testing.h")
    assert set(names) == set(capi.TESTING_EXPORTS)
    for n in names:
        assert not hasattr(lib, n), f"{n} is a testing aid and must not be in the production library"
    with capi.testing_library() as T:
        for n in names + list(capi.EXPORTS):
            assert hasattr(T, n), n
    assert capi.lib() is lib


def test_draw_is_the_reference_generator(lib, golden):
    from molla_b200 import capi
    for s, c, v in zip(golden["draw_seed"], golden["draw_counter"], golden["draw_value"]):
        assert np.float32(capi.draw(int(s), int(c))) == v


def test_argument_errors_come_before_any_launch(lib):
    from molla_b200 import capi
    null = C.c_void_p(None)
    args = [null, 0, 1, 1] + [null] * 16 + [0, null, 0, null] + [null] * 6
    assert lib.molla_sample_batch(*args) == capi.ERR_ARGUMENT
    assert "required" in capi.last_error()
    assert lib.molla_sample_workspace_bytes(-1, 10, 0) == capi.ERR_ARGUMENT
    assert lib.molla_sample_workspace_bytes(1, 0, 0) == capi.ERR_ARGUMENT
    assert lib.molla_sample_workspace_bytes(1, 10, 21) == capi.ERR_ARGUMENT
    assert lib.molla_sample_logprobs(null, 0, 1, 1, null, null) == capi.ERR_ARGUMENT
    assert lib.molla_sample_expf(null, 1, null, null) == capi.ERR_ARGUMENT


def test_host_entry_validates_settings_like_the_reference(lib):
    """SamplerConfig.check (sample.mojo:140-154): refused on the host, nothing launched."""
    from molla_b200 import capi
    B, V = 2, 8
    logits = np.zeros((B, V), np.float32)
    tok = np.zeros(B, np.int32)
    st = np.zeros(B, np.uint32)
    p = lambda a: C.c_void_p(a.ctypes.data)
    null = C.c_void_p(None)

    def call(temperature, top_k=None, top_p=None, rp=None, bias=None):
        t = np.asarray(temperature, np.float32)
        k = None if top_k is None else np.asarray(top_k, np.int32)
        tp = None if top_p is None else np.asarray(top_p, np.float32)
        r = None if rp is None else np.asarray(rp, np.float32)
        bi = bv = bo = None
        if bias is not None:
            bi, bv, bo = np.array([bias], np.int64), np.array([1.0], np.float32), np.array([0, 1, 1], np.int32)
        q = lambda a: null if a is None else p(a)
        keep = (t, k, tp, r, bi, bv, bo)
        rc = lib.molla_sample_batch_host(
            p(logits), V, B, V, p(t), q(k), q(tp), null, null, q(r), null, null, null, null, null, null, null,
            q(bi), q(bv), q(bo), 0, null, 0, null, p(tok), null, null, null, p(st))
        del keep
        return rc, capi.last_error()

    assert call([-1.0, 0.0]) == (capi.ERR_CONFIG, "a temperature cannot be negative")
    assert call([0.0, 0.0], top_k=[0, -3]) == (capi.ERR_CONFIG, "a top-k cannot be negative")
    assert call([0.0, 0.0], top_p=[0.0, 1.0])[0] == capi.ERR_CONFIG
    assert call([0.0, 0.0], top_p=[1.5, 1.0])[0] == capi.ERR_CONFIG
    assert call([0.0, 0.0], rp=[1.0, 0.0])[0] == capi.ERR_CONFIG
    assert call([0.0, 0.0], bias=V)[0] == capi.ERR_CONFIG  # a bias outside the vocabulary
    # ragged lists: offsets that go backwards are refused before anything is sized by them
    t = np.zeros(B, np.float32)
    hist = np.zeros(4, np.int64)
    bad = np.array([0, 3, 1], np.int32)
    rc = lib.molla_sample_batch_host(
        p(logits), V, B, V, p(t), null, null, null, null, null, null, null, null, null, null, p(hist), p(bad),
        null, null, null, 0, null, 0, null, p(tok), null, null, null, p(st))
    assert rc == capi.ERR_ARGUMENT and "non-decreasing" in capi.last_error()
