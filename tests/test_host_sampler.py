"""Host side of the sampler (no GPU): settings validation, the penalty ring, the
per-row arrays handed to the C entry point."""
import numpy as np
import pytest

from molla_b200.sampler import Sampler, SamplerConfig, params_of


def test_defaults_are_the_references():
    c = SamplerConfig()
    assert (c.temperature, c.top_k, c.top_p, c.min_p, c.typical_p) == (0.0, 0, 1.0, 0.0, 1.0)
    assert (c.repeat_penalty, c.frequency_penalty, c.presence_penalty, c.repeat_last_n, c.seed) == (1.0, 0.0, 0.0, 64, 0)
    assert c.greedy() and not c.penalizing()
    assert SamplerConfig(frequency_penalty=0.1).penalizing()
    assert not SamplerConfig(frequency_penalty=0.1, repeat_last_n=0).penalizing()


@pytest.mark.parametrize("kw,msg", [
    (dict(temperature=-1.0), "a temperature cannot be negative"),
    (dict(top_k=-1), "a top-k cannot be negative"),
    (dict(top_p=0.0), "a top-p has to be above zero and at most one"),
    (dict(top_p=1.5), "a top-p has to be above zero and at most one"),
    (dict(min_p=-0.1), "a min-p has to be between zero and one"),
    (dict(min_p=1.1), "a min-p has to be between zero and one"),
    (dict(typical_p=0.0), "a typical-p has to be above zero and at most one"),
    (dict(repeat_penalty=0.0), "a repetition penalty of zero or less erases a logit"),
    (dict(repeat_last_n=-1), "a penalty window cannot be negative"),
])
def test_check_refuses_what_the_reference_refuses(kw, msg):
    with pytest.raises(ValueError, match=msg):
        Sampler(SamplerConfig(**kw), 5, device="cpu")


def test_vocabulary_and_bias_errors():
    with pytest.raises(ValueError, match="a sampler needs a vocabulary"):
        Sampler(SamplerConfig(), 0, device="cpu")
    s = Sampler(SamplerConfig(), 5, device="cpu")
    with pytest.raises(ValueError, match="a logit bias names token 5"):
        s.bias(5, 1.0)
    with pytest.raises(ValueError):
        s.bias(-1, 1.0)
    s.bias(2, 1.0)
    assert s.biasing()


def test_ring_window_forgets_and_resets():
    s = Sampler(SamplerConfig(frequency_penalty=0.2, repeat_last_n=2), 5, device="cpu")
    for t in (0, 1, 1):
        s.observe(t)
    assert (s.count_of(0), s.count_of(1), s.filled) == (0, 2, 2)
    s._took(3)
    assert s.drawn == 1 and s.count_of(3) == 1 and s.count_of(1) == 1
    s.reset()
    assert (s.filled, s.drawn, s.head) == (0, 0, 0)
    off = Sampler(SamplerConfig(frequency_penalty=0.2, repeat_last_n=0), 5, device="cpu")
    off.observe(0)
    assert off.filled == 0 and off.count_of(0) == 0


def test_params_of_lays_out_parallel_arrays():
    a = Sampler(SamplerConfig(temperature=0.7, top_k=40, seed=9), 100, device="cpu")
    b = Sampler(SamplerConfig(repeat_last_n=0, seed=2**64 - 1), 100, device="cpu")
    for t in (5, 6, 5):
        a.observe(t)
    a.bias(3, -1.0)
    b.drawn = 7
    w = params_of([a, b])
    assert w["temperature"].dtype == np.float32 and w["top_k"].tolist() == [40, 0]
    assert w["hist"].tolist() == [5, 6, 5] and w["hist_off"].tolist() == [0, 3, 3]
    assert w["window_on"].tolist() == [1, 0]
    assert w["bias_ids"].tolist() == [3] and w["bias_off"].tolist() == [0, 1, 1]
    assert w["seed"].tolist() == [9, 2**64 - 1] and w["drawn"].tolist() == [0, 7]
