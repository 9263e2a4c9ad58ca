"""The logprob fields of the OpenAI request and response shapes, for the outputs this library
adds to the sampling step (the chosen token's logprob and the top-N logprobs of the raw logits).

The reference parses requests in src/molla/api/openai.mojo and today refuses `logprobs` and
`top_logprobs` (`_refuse_unsupported`, :156-161) and writes `"logprobs": null` into every
completion choice (`_write_text_choice`, :645). This module is the host-side counterpart for a
build that samples with this library: which request fields switch the outputs on
(`read_logprob_request`, same validation order and refusal style), and the two response objects
(`chat_logprobs`, `completion_logprobs`). Token ids become text through a caller-supplied
`decode(token_id) -> bytes`: the tokenizer is outside this library.
"""
from __future__ import annotations

from typing import Callable, Mapping, Sequence

TOP_LOGPROBS_MAX = 20  # the API's limit, and the library's TOPN_MAX


def read_logprob_request(body: Mapping, chat: bool) -> tuple[bool, int]:
    """(want_logprob, top_n) of a request body.

    Chat completions: `logprobs` is a boolean, `top_logprobs` an integer 0..20 that needs
    `logprobs: true`. Legacy completions: `logprobs` is an integer 0..5 asking for that many
    alternatives (0 = the chosen token's only)."""
    lp = body.get("logprobs")
    top = body.get("top_logprobs")
    if chat:
        if lp is not None and not isinstance(lp, bool):
            raise ValueError("logprobs has to be true or false")
        if top is not None:
            if isinstance(top, bool) or not isinstance(top, int) or not 0 <= top <= TOP_LOGPROBS_MAX:
                raise ValueError("top_logprobs has to be an integer between 0 and 20")
            if not lp:
                raise ValueError("top_logprobs needs logprobs to be true")
        return bool(lp), int(top or 0) if lp else 0
    if top is not None:
        raise ValueError("top_logprobs belongs to chat completions; completions take an integer logprobs")
    if lp is None:
        return False, 0
    if isinstance(lp, bool) or not isinstance(lp, int) or not 0 <= lp <= 5:
        raise ValueError("logprobs has to be an integer between 0 and 5")
    return True, int(lp)


def _text(b: bytes) -> str:
    return b.decode("utf-8", "replace")


def _entry(tok: int, lp: float, decode: Callable[[int], bytes]) -> dict:
    b = decode(int(tok))
    return {"token": _text(b), "logprob": float(lp), "bytes": list(b)}


def chat_logprobs(tokens: Sequence[int], chosen_logprobs: Sequence[float], top_ids, top_logprobs,
                  decode: Callable[[int], bytes]) -> dict:
    """`choices[i].logprobs` of a chat completion: one entry per generated token with its text,
    logprob and bytes, and under `top_logprobs` the alternatives in descending logprob (ties to
    the lower token id, as the library orders them). Slots the library padded with -1 are left out."""
    content = []
    for i, (t, lp) in enumerate(zip(tokens, chosen_logprobs)):
        e = _entry(t, lp, decode)
        alts = []
        if top_ids is not None:
            for a, alp in zip(top_ids[i], top_logprobs[i]):
                if int(a) >= 0:
                    alts.append(_entry(a, alp, decode))
        e["top_logprobs"] = alts
        content.append(e)
    return {"content": content}


def completion_logprobs(tokens: Sequence[int], chosen_logprobs: Sequence[float], top_ids, top_logprobs,
                        decode: Callable[[int], bytes], text_offset0: int = 0) -> dict:
    """`choices[i].logprobs` of a legacy completion: parallel arrays `tokens`, `token_logprobs`,
    `top_logprobs` (one {text: logprob} map per token, or null when none were asked for) and
    `text_offset` (character offsets into the returned text)."""
    toks, lps, tops, offs = [], [], [], []
    at = text_offset0
    for i, (t, lp) in enumerate(zip(tokens, chosen_logprobs)):
        s = _text(decode(int(t)))
        toks.append(s); lps.append(float(lp)); offs.append(at)
        at += len(s)
        if top_ids is None:
            tops.append(None)
        else:
            m = {}
            for a, alp in zip(top_ids[i], top_logprobs[i]):
                if int(a) >= 0:
                    m.setdefault(_text(decode(int(a))), float(alp))  # two ids with one text: the likelier comes first
            tops.append(m)
    return {"tokens": toks, "token_logprobs": lps, "top_logprobs": tops, "text_offset": offs}
