"""CPU-side checks of the product library: it loads, exports every symbol the header declares, and its
host integer logic is bit-identical to the oracle. No compute kernel runs here."""
import re
from pathlib import Path

import numpy as np
import pytest
from hypothesis import given, settings, strategies as st

ROOT = Path(__file__).resolve().parent.parent


def test_library_exports_every_declared_symbol(dcd):
    from decidra_b200 import _lib
    header = (ROOT / "include" / "decidra_b200.h").read_text()
    declared = set(re.findall(r"DCD_API\s+[\w\s\*]+?\b(dcd_\w+)\s*\(", header))
    assert len(declared) >= 50
    lib = _lib.load()
    for name in sorted(declared):
        assert hasattr(lib, name), f"{name} declared in the header but not exported"
    assert declared == set(_lib.SIGNATURES), declared ^ set(_lib.SIGNATURES)


def test_engine_create_fails_loudly_without_gpu(dcd):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(dcd.EngineError) as ei:
        dcd.Engine(dcd.tiny_config())
    assert ei.value.code == 4 and "CUDA" in str(ei.value)


def test_create_rejects_bad_config(dcd):
    from decidra_b200 import _lib
    import ctypes as C
    cfg = dcd.tiny_config()
    cfg.conv_kernel = 3
    out = C.c_void_p()
    rc = _lib.load().dcd_engine_create(C.byref(cfg), None, 0, C.byref(out))
    assert rc == 3 and not out.value and b"conv" in _lib.load().dcd_last_error(None)
    opt = dcd.Options()
    opt.precision = 7
    rc = _lib.load().dcd_engine_create(C.byref(dcd.tiny_config()), C.byref(opt), 0, C.byref(out))
    assert rc == 3 and b"unknown" in _lib.load().dcd_last_error(None)
    opt.precision = 2   # quantised precisions need a bf16 engine; tiny_config() is f32
    rc = _lib.load().dcd_engine_create(C.byref(dcd.tiny_config()), C.byref(opt), 0, C.byref(out))
    assert rc == 3 and b"bf16 engine" in _lib.load().dcd_last_error(None)


@settings(max_examples=200, deadline=None)
@given(lens=st.lists(st.integers(1, 600), min_size=1, max_size=300), state=st.integers(2, 20000),
       rows=st.integers(1, 80), keys=st.integers(1 << 10, 1 << 20), scores=st.integers(1 << 14, 1 << 28))
def test_plan_chunks_bit_exact_vs_oracle(dcd, oracle, lens, state, rows, keys, scores):
    from decidra_b200 import answers
    try:
        want = oracle.plan_chunks(lens, state, rows, keys, scores)
    except ValueError:
        with pytest.raises(ValueError):
            answers.plan_chunks(lens, state, rows, keys, scores)
        return
    got = answers.plan_chunks(lens, state, rows, keys, scores)
    assert got[0] == want[0]
    assert (got[1] == want[1]).all() and (got[2] == want[2]).all()


@settings(max_examples=60, deadline=None)
@given(seq=st.integers(2, 70), data=st.data())
def test_mask_bit_exact_vs_oracle(dcd, oracle, seq, data):
    from decidra_b200 import answers
    split = data.draw(st.integers(1, seq - 1))
    assert (answers.block_cascade_mask(seq, split) == oracle.block_cascade_mask(seq, split)).all()
    for bad in (0, seq, seq + 1):
        with pytest.raises(ValueError):
            answers.block_cascade_mask(seq, bad)


@settings(max_examples=300, deadline=None)
@given(logits=st.lists(st.floats(-12, 12, width=32), min_size=2, max_size=255), temp=st.floats(0.0625, 4.0, width=32),
       kind=st.sampled_from(["choice", "noul", "score"]))
def test_decode_answer_bit_exact_vs_oracle(dcd, oracle, logits, temp, kind):
    from decidra_b200 import answers
    try:
        shares_o, out_o = oracle.decode_answer(logits, len(logits), temp, kind)
    except ValueError:  # exp overflow -> "non-finite d3 logits" on both sides
        with pytest.raises(ValueError):
            answers.decode_answer(logits, len(logits), temp, kind)
        return
    shares, value, conf = answers.decode_answer(logits, len(logits), temp, kind)
    assert shares.tobytes() == shares_o.tobytes()
    assert np.float32(value).tobytes() == out_o[0].tobytes() and np.float32(conf).tobytes() == out_o[1].tobytes()


def test_to_answer_shapes(dcd):
    from decidra_b200 import answers
    a = answers.to_answer("choice", ["A", "B", "C"], [0.1, 2.0, -1.0])
    assert a["type"] == "choice" and a["choice"] == "B" and set(a["probabilities"]) == {"A", "B", "C"}
    assert answers.to_answer("noul", ["no", "yes"], [0.0, 0.0])["noul"] == 0.5
    s = answers.to_answer("score", ["0", "1", "2"], [0.0, 0.0, 0.0], texts=["bad", "ok", "good"])
    assert abs(s["score"] - 1.0) < 1e-6 and s["legend"]["2"] == "good"
    with pytest.raises(ValueError):
        answers.decode_answer([1e38, 1e38], 2, 1e-3, "choice")  # exp overflows -> non-finite
