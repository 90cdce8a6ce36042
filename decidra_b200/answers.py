"""Host-side integer/typed-answer logic through the C ABI (no GPU needed).

``decode_answer`` follows ``NativeBackend::answers`` (src/native_backend.rs:611-619) and
``d3::to_answer`` (src/d3.rs:373-438) of juanqui/decidra; ``plan_chunks`` follows
``Engine::state_once_batch_rows`` (native/src/engine.rs:4893-4918); ``block_cascade_mask`` follows
native/src/engine.rs:490-504.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib

KIND = {"choice": 0, "noul": 1, "score": 2}


def decode_answer(logits, count: int, temperature: float, kind: str):
    """Returns (shares[count], value, confidence): value = choice index | noul p[1] | score."""
    logits = np.ascontiguousarray(logits, dtype=np.float32)
    shares = np.zeros(count, np.float32)
    out2 = np.zeros(2, np.float32)
    rc = _lib.load().dcd_decode_answer(logits.ctypes.data_as(_lib.FP), count, temperature, KIND[kind], shares.ctypes.data_as(_lib.FP), out2.ctypes.data_as(_lib.FP))
    if rc:
        raise ValueError("non-finite d3 logits")
    return shares, float(out2[0]), float(out2[1])


def to_answer(kind: str, keys, logits, temperature: float = 1.0, texts=None) -> dict:
    """Typed answer object shaped like the reference's JSON (src/d3.rs:398-437)."""
    shares, value, conf = decode_answer(logits, len(keys), temperature, kind)
    if kind == "score":
        return {"type": "score", "score": value, "probabilities": dict(zip(keys, shares.tolist())), "confidence": conf,
                "legend": dict(zip(keys, texts or keys))}
    if kind == "noul":
        return {"type": "noul", "noul": value}
    return {"type": "choice", "choice": keys[int(value)], "probabilities": dict(zip(keys, shares.tolist())), "confidence": conf}


def plan_chunks(lens, state_len: int, max_rows: int = 64, max_keys: int = 1 << 18, max_scores: int = 1 << 27):
    lens = np.ascontiguousarray(lens, dtype=np.uint64)
    B = lens.size
    order = np.zeros(max(B, 1), np.int32)
    chunk_of = np.zeros(max(B, 1), np.int32)
    n = C.c_int32()
    rc = _lib.load().dcd_plan_chunks(lens.ctypes.data_as(C.POINTER(C.c_size_t)), B, state_len, max_rows, max_keys, max_scores,
                                     order.ctypes.data_as(_lib.I32P), chunk_of.ctypes.data_as(_lib.I32P), C.byref(n))
    if rc:
        raise ValueError("empty batch, zero cap, or one question exceeds the caps")
    return n.value, order[:B], chunk_of[:B]


def block_cascade_mask(seq: int, split: int) -> np.ndarray:
    mask = np.zeros((seq * seq + 7) // 8, dtype=np.uint8)
    rc = _lib.load().dcd_block_cascade_mask(seq, split, mask.ctypes.data_as(C.POINTER(C.c_uint8)))
    if rc:
        raise ValueError(f"block split {split} out of range for {seq} tokens")
    return mask
