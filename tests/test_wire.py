"""The logprob fields of the OpenAI request and response shapes (molla_b200/wire.py): what the
reference's API layer would parse and write once it stops refusing `logprobs`
(src/molla/api/openai.mojo:156-161, :645). Host-only."""
import json

import numpy as np
import pytest

from molla_b200 import wire

VOCAB = {0: b"Hello", 1: b" world", 2: b"!", 3: b"\xe2\x82", 4: b" world"}   # 3: half a code point; 4: same text as 1


def decode(t):
    return VOCAB[t]


def test_request_fields():
    assert wire.read_logprob_request({}, chat=True) == (False, 0)
    assert wire.read_logprob_request({"logprobs": False}, chat=True) == (False, 0)
    assert wire.read_logprob_request({"logprobs": True}, chat=True) == (True, 0)
    assert wire.read_logprob_request({"logprobs": True, "top_logprobs": 5}, chat=True) == (True, 5)
    assert wire.read_logprob_request({"logprobs": 3}, chat=False) == (True, 3)
    assert wire.read_logprob_request({"logprobs": 0}, chat=False) == (True, 0)
    for body, chat in (({"logprobs": 1}, True), ({"top_logprobs": 3}, True), ({"logprobs": True, "top_logprobs": 21}, True),
                       ({"logprobs": True, "top_logprobs": True}, True), ({"logprobs": 6}, False),
                       ({"logprobs": True}, False), ({"logprobs": 1, "top_logprobs": 1}, False)):
        with pytest.raises(ValueError):
            wire.read_logprob_request(body, chat)


def test_chat_object():
    top_ids = np.array([[0, 1, -1], [1, 4, 2]], np.int32)
    top_lps = np.array([[-0.1, -2.5, 0.0], [-0.7, -0.7, -3.0]], np.float32)
    out = wire.chat_logprobs([0, 3], [-0.1, -4.0], top_ids, top_lps, decode)
    json.dumps(out)
    c = out["content"]
    assert [e["token"] for e in c] == ["Hello", "�"] and c[1]["bytes"] == [0xE2, 0x82]
    assert abs(c[0]["logprob"] + 0.1) < 1e-6
    assert [a["token"] for a in c[0]["top_logprobs"]] == ["Hello", " world"]         # the padded slot is gone
    assert [a["bytes"] for a in c[1]["top_logprobs"]][0] == list(b" world") and len(c[1]["top_logprobs"]) == 3
    assert wire.chat_logprobs([2], [-1.0], None, None, decode)["content"][0]["top_logprobs"] == []


def test_completion_object():
    top_ids = np.array([[0, 1], [1, 4]], np.int32)
    top_lps = np.array([[-0.1, -2.5], [-0.7, -0.9]], np.float32)
    out = wire.completion_logprobs([0, 1], [-0.1, -0.7], top_ids, top_lps, decode, text_offset0=3)
    json.dumps(out)
    assert out["tokens"] == ["Hello", " world"] and out["text_offset"] == [3, 8]
    assert out["top_logprobs"][1] == {" world": pytest.approx(-0.7)}                 # one text, the likelier id
    assert wire.completion_logprobs([2], [-1.0], None, None, decode)["top_logprobs"] == [None]
