"""Pins the CPU oracle: the reference's own unit-test vectors for the integer/layout parts, and
structural properties of the floating-point path (state-once == per-row, negative controls)."""
import numpy as np
import pytest

from conftest import orc_cfg, tiny_inputs
from decidra_b200.config import tiny_config


# ---- reference golden: native/src/engine.rs:5499-5522 (mask_tests) ------------------------------
def _bit(mask, seq, q, k):
    i = q * seq + k
    return bool(mask[i // 8] & (1 << (i % 8)))


def test_block_cascade_state_never_sees_question(oracle):
    seq, split = 11, 5
    m = oracle.block_cascade_mask(seq, split)
    assert len(m) == (seq * seq + 7) // 8
    for q in range(seq):
        for k in range(seq):
            assert _bit(m, seq, q, k) == ((k < split) if q < split else True), (q, k)
    assert not _bit(m, seq, 0, split)
    assert not _bit(m, seq, split - 1, seq - 1)
    assert _bit(m, seq, split, 0)
    assert _bit(m, seq, split, seq - 1)


def test_block_cascade_split_bounds(oracle):
    for split in (0, 5, 6):
        with pytest.raises(ValueError):
            oracle.block_cascade_mask(5, split)


# ---- reference golden: native/src/weights.rs:833-847 (nvfp4_scale_repack_uses_cublaslt_tiles) ----
def test_nvfp4_scale_repack_tiles(oracle):
    outer, inner = 3, 128
    src = np.arange(outer * inner // 16, dtype=np.uint8)
    got = oracle.repack_nvfp4_scales(src, outer, inner)
    assert len(got) == (inner // 64) * 1 * 512
    for o in range(outer):
        for j in range(inner // 16):
            base = ((j // 4) + (o // 128) * (inner // 64)) * 512
            off = base + (o % 32) * 16 + ((o % 128) // 32) * 4 + (j % 4)
            assert got[off] == src[o * (inner // 16) + j]


# ---- reference golden: src/d3.rs:520-526 (choice_confidence_matches_the_serving_contract) ---------
def test_choice_confidence_known_answers(oracle):
    # feed probabilities as logits = log p with T = 1 so that the decoded shares are those probabilities
    for probs, want, tol in (([0.9996, 0.00004, 0.0003], 0.9994, 1e-3), ([0.030755, 0.152012, 0.817233], 0.72585, 1e-4)):
        shares, out2 = oracle.decode_answer(np.log(np.array(probs, np.float32)), 3, 1.0, "choice")
        assert abs(out2[1] - want) < tol
        assert int(out2[0]) == int(np.argmax(probs))
    shares, out2 = oracle.decode_answer(np.array([0.3], np.float32), 1, 1.0, "choice")
    assert out2[1] == 1.0 and shares[0] == 1.0


def test_decode_score_and_noul(oracle):
    logits = np.array([0.0, 1.0, 2.0, 0.5], np.float32)
    shares, out2 = oracle.decode_answer(logits, 4, 0.7, "score")
    e = np.exp(logits / np.float32(0.7)).astype(np.float32)
    p = e / e.sum(dtype=np.float32)
    assert np.allclose(shares, p, rtol=1e-6)
    assert abs(out2[0] - float((np.arange(4) * p).sum())) < 1e-5
    assert 0.0 <= out2[1] <= 1.0
    shares, out2 = oracle.decode_answer(logits, 2, 1.0, "noul")
    assert out2[0] == shares[1]
    with pytest.raises(ValueError):
        oracle.decode_answer(np.array([1e30, 0], np.float32), 2, 1e-30, "choice")


# ---- chunk planner: native/src/engine.rs:4893-4918 ------------------------------------------------
def test_plan_chunks_reference_caps(oracle):
    # 70 questions under the 64-row cap -> 2 chunks, sorted by length, stable
    lens = [50 + (i * 7) % 9 for i in range(70)]
    n, order, chunk_of = oracle.plan_chunks(lens, 2048)
    assert n == 2
    assert list(order) == sorted(range(70), key=lambda i: lens[i])
    assert (np.bincount(chunk_of) == [64, 6]).all()
    # key cap: rows*(state+maxlen) <= 2^18 with state 16384 -> at most 15 questions of 512
    n, order, chunk_of = oracle.plan_chunks([512] * 40, 16384)
    assert np.bincount(chunk_of).max() == (1 << 18) // (16384 + 512)
    # a single question over the caps is an error
    with pytest.raises(ValueError):
        oracle.plan_chunks([600], 1 << 18)
    with pytest.raises(ValueError):
        oracle.plan_chunks([], 10)


def test_pack_matches_numpy(oracle):
    lens = np.array([16, 1, 33, 7, 64], np.int32)
    cu, pos, tq, last = oracle.pack(lens, 2048)
    assert list(cu) == [0, 16, 17, 50, 57, 121]
    assert list(last) == [15, 16, 49, 56, 120]
    assert (pos == np.concatenate([2048 + np.arange(n) for n in lens])).all()
    assert (tq == np.repeat(np.arange(5), lens)).all()
    with pytest.raises(ValueError):
        oracle.pack([3, 0, 2], 0)
    with pytest.raises(ValueError):
        oracle.pack([], 0)


# ---- committed fixture --------------------------------------------------------------------------
@pytest.mark.parametrize("name,dt", [("f32", 0), ("bf16", 1)])
def test_oracle_matches_committed_fixture(oracle, name, dt):
    from pathlib import Path
    g = np.load(Path(__file__).parent / "golden" / "tiny_oracle.npz")
    qs = np.split(g["questions"], np.cumsum(g["qlens"])[:-1])
    o = oracle.Oracle(orc_cfg(oracle, tiny_config(dt)), 0)
    st = o.capture_state(g["state"])
    got = o.readout_state_once_batch(st, qs)
    np.testing.assert_allclose(got, g[f"logits_{name}"], rtol=0, atol=2e-6 if dt == 0 else 0)
    np.testing.assert_allclose(st.tensor(0, 2), g[f"gdn_state0_{name}"], rtol=0, atol=1e-6)


# ---- structure of the floating-point path (designs of native/tests/d3_state_once*.rs) ------------
@pytest.mark.parametrize("dt", [0, 1])
def test_state_once_equals_per_row_and_negative_controls(oracle, dt):
    state, questions = tiny_inputs()
    o = oracle.Oracle(orc_cfg(oracle, tiny_config(dt)), 0)
    st = o.capture_state(state)
    batch = o.readout_state_once_batch(st, questions)
    assert batch.shape == (4, 255) and np.isfinite(batch).all()
    for i, q in enumerate(questions):
        ref = o.decision_logits_split(np.concatenate([state, q]), len(state))
        np.testing.assert_allclose(batch[i], ref, atol=1e-5)
        single = o.readout_state_once_batch(st, [q])
        np.testing.assert_array_equal(single[0], batch[i])  # batch-shape invariance
    # zeroing the layer-0 recurrent seed or conv tail must move the answer
    st.zero(0, 2)
    assert np.abs(o.readout_state_once_batch(st, questions) - batch).max() > 1e-3
    st2 = o.capture_state(state)
    st2.zero(0, 3)
    assert np.abs(o.readout_state_once_batch(st2, questions) - batch).max() > 1e-3


def test_oracle_rejects_bad_inputs(oracle):
    o = oracle.Oracle(orc_cfg(oracle, tiny_config(0)), 0)
    with pytest.raises(ValueError):
        o.capture_state([5])  # a state needs at least two tokens
    with pytest.raises(ValueError):
        o.capture_state([1, 4096])  # token id out of vocabulary
    st = o.capture_state([1, 2, 3])
    with pytest.raises(ValueError):
        o.readout_state_once_batch(st, [])
    with pytest.raises(ValueError):
        o.readout_state_once_batch(st, [[1, 2], []])
    with pytest.raises(ValueError):
        o.decision_logits_split([1, 2, 3], 3)


def test_generator_statistics(oracle):
    w = oracle.gen_tensor(0, 3, 12, 1 << 18, bf16=False)
    assert abs(w.mean()) < 2e-4 and abs(w.std() - 0.02) < 3e-4
    a = oracle.gen_tensor(0, 0, 36, 4096, bf16=False)
    assert a.min() >= 0 and a.max() <= 2.7725887
    # streaming: a range generated from an offset equals the slice of the whole
    assert (oracle.gen_tensor(0, 3, 12, 100, bf16=True, first=1000) == oracle.gen_tensor(0, 3, 12, 1100, bf16=True)[1000:]).all()
    assert (oracle.rb(w) == np.array([oracle.lib().orc_k_rb(float(v)) for v in w[:256]] + list(oracle.rb(w)[256:]), np.float32)).all()


def test_nvfp4_scale_repack_uses_cublaslt_tiles(oracle):
    """The reference's own known-answer test (native/src/weights.rs:833-847): outer = 3, inner = 128, src[i] = i."""
    outer, inner = 3, 128
    src = np.arange(outer * inner // 16, dtype=np.uint8).reshape(outer, inner // 16)
    got = oracle.nvfp4_scale_repack(src, inner)
    assert got.size == (inner // 64) * 1 * 512
    for o in range(outer):
        for j in range(inner // 16):
            base = ((j // 4) + (o // 128) * (inner // 64)) * 512
            off = base + (o % 32) * 16 + ((o % 128) // 32) * 4 + (j % 4)
            assert got[off] == src[o, j], (o, j)
    assert int(got.astype(np.int64).sum()) == int(src.astype(np.int64).sum())   # everything else is padding
