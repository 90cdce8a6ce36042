"""d3 prompt contract over the C ABI: the host-side mirror of juanqui/decidra's ``src/d3.rs`` (text path)
and ``src/pyjson.rs``. The rendering itself is C++ (``csrc/prompt.cpp``); JSON values cross the boundary as
text with their key order intact.
"""
from __future__ import annotations

import ctypes as C
import json
from typing import Sequence

from . import _lib
from .engine import EngineError


def _err() -> str:
    return (_lib.load().dcd_prompt_last_error() or b"").decode("utf-8", "replace")


def _text(call, *args) -> str:
    """Run a text-producing entry point: size query, then the real call."""
    need = C.c_size_t()
    cap = 1024
    while True:
        buf = C.create_string_buffer(cap)
        rc = call(*args, buf, cap, C.byref(need))
        if rc == 0:
            return buf.raw[:need.value].decode("utf-8")
        if need.value + 1 > cap and _err() == "output buffer too small":
            cap = need.value + 1
            continue
        raise EngineError(rc, _err())


def _doc(value) -> bytes:
    return json.dumps(value, ensure_ascii=True).encode()


def format_float(value: float) -> str:
    """``pyjson::format_float``: CPython's ``repr(float)``."""
    return _text(_lib.load().dcd_format_float, C.c_double(value))


def dumps(value) -> str:
    """``pyjson::dumps``: ``json.dumps(value, ensure_ascii=False)`` byte for byte."""
    d = _doc(value)
    return _text(_lib.load().dcd_pyjson_dumps, d, len(d))


def dumps_text(json_text: str) -> str:
    """``dumps`` of a JSON document given as text (number literals are classified as serde_json does)."""
    d = json_text.encode()
    return _text(_lib.load().dcd_pyjson_dumps, d, len(d))


def py_repr(value) -> str:
    d = _doc(value)
    return _text(_lib.load().dcd_pyjson_repr, d, len(d), 0)


def py_str(value) -> str:
    d = _doc(value)
    return _text(_lib.load().dcd_pyjson_repr, d, len(d), 1)


def py_truthy(value) -> bool:
    d = _doc(value)
    out = C.c_int()
    rc = _lib.load().dcd_pyjson_truthy(d, len(d), C.byref(out))
    if rc:
        raise EngineError(rc, _err())
    return bool(out.value)


def parse_question(question) -> dict:
    """``d3::parse_question``: {"kind", "instructions", "keys", "texts"}."""
    d = _doc(question)
    return json.loads(_text(_lib.load().dcd_d3_parse_question, d, len(d)))


def render(state, question, codes: Sequence[str]) -> str:
    """``d3::render`` of a parsed-on-the-fly question object."""
    s, q = _doc(state), _doc(question)
    arr = (C.c_char_p * max(len(codes), 1))(*[c.encode() for c in codes])
    return _text(_lib.load().dcd_d3_render, s, len(s), q, len(q), arr, len(codes))


def state_end_char(text: str, state) -> int:
    """``d3::state_end_char``: byte offset of the end of the state segment in the UTF-8 prompt."""
    t, s = text.encode(), _doc(state)
    out = C.c_size_t()
    rc = _lib.load().dcd_d3_state_end_char(t, len(t), s, len(s), C.byref(out))
    if rc:
        raise EngineError(rc, _err())
    return out.value


def char_to_byte_offsets(text: str, offsets: Sequence[tuple]) -> list:
    """Character offsets (what HF ``tokenizers`` reports in Python) -> UTF-8 byte offsets (what the Rust tokenizer of the
    reference reports and what ``state_end_char`` / ``state_token_count`` work in). Identity for ASCII text."""
    at = [0]
    for ch in text:
        at.append(at[-1] + len(ch.encode("utf-8")))
    return [(at[a], at[b]) for a, b in offsets]


def state_token_count(offsets: Sequence[tuple], end_char: int) -> int:
    """``d3::state_token_count``: the state/question split from tokenizer offsets. ``offsets`` and ``end_char`` are UTF-8 BYTE
    offsets into the prompt, as in the reference (Rust ``tokenizers`` offsets index the ``&str`` bytes); offsets from a Python
    tokenizer are character offsets and go through ``char_to_byte_offsets`` first."""
    flat = (C.c_size_t * max(2 * len(offsets), 1))(*[v for pair in offsets for v in pair])
    out = C.c_size_t()
    rc = _lib.load().dcd_d3_state_token_count(flat, len(offsets), end_char, C.byref(out))
    if rc:
        raise EngineError(rc, _err())
    return out.value


def contains_media(state) -> bool:
    s = _doc(state)
    out = C.c_int()
    rc = _lib.load().dcd_d3_contains_media(s, len(s), C.byref(out))
    if rc:
        raise EngineError(rc, _err())
    return bool(out.value)
