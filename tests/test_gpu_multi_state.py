"""One question pass over questions of several states: rows must equal, bit for bit, those of one
`readout_state_once_batch` call per state (same kernels, same per-row arithmetic; only the batching differs)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _mixed(cfg_vocab, rng, state_lens, n_questions, qlo, qhi):
    states = [rng.integers(0, cfg_vocab, n, dtype=np.uint32) for n in state_lens]
    state_of = rng.integers(0, len(states), n_questions).astype(np.uint32)
    state_of[: len(states)] = np.arange(len(states))          # every state gets at least one question
    rng.shuffle(state_of)
    questions = [rng.integers(0, cfg_vocab, int(n), dtype=np.uint32) for n in rng.integers(qlo, qhi + 1, n_questions)]
    return states, state_of, questions


def _check(e, states, state_of, questions):
    caches = [e.capture_state(s) for s in states]
    got = e.readout_multi_state_batch(caches, questions, state_of)
    assert got.shape == (len(questions), e.cfg.readout_rows) and np.isfinite(got).all()
    for k, c in enumerate(caches):
        idx = [i for i in range(len(questions)) if state_of[i] == k]
        want = e.readout_state_once_batch(c, [questions[i] for i in idx])
        assert got[idx].tobytes() == want.tobytes(), k
    # the answers depend on the state: two states give different rows for the same question
    if len(states) > 1:
        a = e.readout_state_once_batch(caches[0], [questions[0]])
        b = e.readout_state_once_batch(caches[1], [questions[0]])
        assert not np.array_equal(a, b)
    return got


@pytest.mark.parametrize("dtype", [0, 1])
def test_multi_state_pass_tiny(dcd, dtype):
    """Tiny configuration: the FMA attention, chunked / sequential GDN and scalar conv kernels on group slices."""
    cfg = dcd.tiny_config(dtype)
    o = dcd.Options()
    o.max_pass_tokens = 1024
    e = dcd.Engine(cfg, o)
    e.init_random(0)
    rng = np.random.default_rng(21)
    states, state_of, questions = _mixed(cfg.vocab, rng, [128, 37, 2, 200], 19, 1, 40)
    _check(e, states, state_of, questions)
    # one state only, and a state that no question names
    _check(e, states[:1], np.zeros(5, np.uint32), questions[:5])
    caches = [e.capture_state(s) for s in states[:3]]
    got = e.readout_multi_state_batch(caches, questions[:4], [2, 2, 0, 2])
    want = e.readout_state_once_batch(caches[2], [questions[0], questions[1], questions[3]])
    assert got[[0, 1, 3]].tobytes() == want.tobytes()
    with pytest.raises(dcd.EngineError, match="names state 3 of 3"):
        e.readout_multi_state_batch(caches, questions[:2], [0, 3])
    with pytest.raises(dcd.EngineError, match="has no tokens"):
        e.readout_multi_state_batch(caches, [questions[0], []], [0, 1])
    with pytest.raises(dcd.EngineError, match="exceeds max_pass_tokens"):
        e.readout_multi_state_batch(caches, [rng.integers(0, cfg.vocab, 1100, dtype=np.uint32)] * 2, [0, 1])
    # a batch larger than the workspace (1024 tokens) runs as several passes, cut inside a state's run of questions too
    big_q = [rng.integers(0, cfg.vocab, int(n), dtype=np.uint32) for n in rng.integers(60, 200, 30)]
    big_of = rng.integers(0, 3, 30).astype(np.uint32)
    assert sum(len(q) for q in big_q) > 2 * 1024
    got = e.readout_multi_state_batch(caches, big_q, big_of)
    for k in range(3):
        idx = [i for i in range(30) if big_of[i] == k]
        for i in idx:   # one by one: the per-state chunk planner is not part of this comparison
            assert got[i].tobytes() == e.readout_state_once_batch(caches[k], [big_q[i]])[0].tobytes(), i
    e.close()


def test_multi_state_pass_d3_slice(dcd):
    """d3-shaped 4-layer slice: the tcgen05 attention (per-group tile tables and state descriptors), the tcgen05 GDN
    (per-group seed) and the vectorised conv on group slices; state lengths on both sides of the 128-key tile."""
    cfg = dcd.d3_config(num_layers=4, vocab=4096)
    o = dcd.Options()
    o.max_pass_tokens = 4096
    e = dcd.Engine(cfg, o)
    e.init_random(3)
    rng = np.random.default_rng(5)
    states, state_of, questions = _mixed(cfg.vocab, rng, [300, 128, 65, 513], 24, 17, 150)
    _check(e, states, state_of, questions)
    e.close()


@pytest.mark.parametrize("precision", [1, 3])
def test_multi_state_pass_quantised_engines(dcd, precision):
    """W4A16 and native NVFP4 engines: weights and activations are quantised row by row (per token, per output row),
    so a row's answer cannot depend on which other questions share the pass."""
    cfg = dcd.d3_config(num_layers=4, vocab=4096)
    o = dcd.Options()
    o.max_pass_tokens = 2048
    o.precision = precision
    e = dcd.Engine(cfg, o)
    e.init_random(3)
    rng = np.random.default_rng(8)
    states, state_of, questions = _mixed(cfg.vocab, rng, [200, 129], 10, 20, 120)
    _check(e, states, state_of, questions)
    e.close()


@pytest.mark.parametrize("which", ["tiny_f32", "tiny_bf16", "d3_slice", "d3_slice_stream_order", "d3_slice_nvfp4", "d3_slice_w4a16"])
def test_cold_request_in_one_pass_is_bit_identical_to_capture_then_readout(dcd, which):
    """dcd_capture_and_readout: the state rides in the same pass as its questions. Logits and every tensor of the returned cache
    must equal those of capture_state + readout_state_once_batch bit for bit, on the fallback kernels (tiny model) and on the
    tensor-core kernels (d3-shaped slice, also with NVFP4 and W4A16 weights); the cache must serve a later warm request. On the
    d3-shaped slice the state's delta rule runs on a second stream beside the questions' conv and preparation (state lengths that
    are not a multiple of the 64-token chunk make its last chunk read rows the other stream is writing, masked in the kernel);
    "stream_order" switches that off (gdn_overlap = 1)."""
    if which.startswith("tiny"):
        cfg = dcd.tiny_config(0 if which == "tiny_f32" else 1)
        vocab, cases = cfg.vocab, [(128, (16, 20, 24, 32)), (2, (1,)), (67, (5, 64, 3))]
    else:
        cfg = dcd.d3_config(num_layers=4, dtype=1, vocab=4096)
        vocab, cases = 4096, [(160, (20, 33, 24, 40)), (300, (130, 7)), (64, (64,))]
    opt = dcd.Options()
    opt.max_pass_tokens = 1024
    opt.precision = {"d3_slice_nvfp4": 3, "d3_slice_w4a16": 1}.get(which, 0)
    opt.gdn_overlap = 1 if which == "d3_slice_stream_order" else 0
    e = dcd.Engine(cfg, opt)
    e.init_random(0)
    rng = np.random.Generator(np.random.PCG64(11))
    for S, qlens in cases:
        state = rng.integers(0, vocab, S, dtype=np.uint32)
        qs = [rng.integers(0, vocab, n, dtype=np.uint32) for n in qlens]
        st_a = e.capture_state(state)
        want = e.readout_state_once_batch(st_a, qs)
        st_b, got = e.capture_and_readout(state, qs)
        assert got.tobytes() == want.tobytes(), (which, S, qlens, float(np.abs(got - want).max()))
        assert st_b.state_len == S and st_b.nbytes == st_a.nbytes
        for li in range(cfg.num_layers):
            for kind in range(4):
                a, b = st_a.tensor(li, kind), st_b.tensor(li, kind)
                assert (a is None) == (b is None)
                if a is not None:
                    assert a.tobytes() == b.tobytes(), (which, S, li, kind)
        warm = e.readout_state_once_batch(st_b, qs[:1])
        assert warm.tobytes() == want[:1].tobytes()
        if which == "d3_slice" and S % 64:  # the two streams race on nothing: the same bits every time
            for _ in range(8):
                st_c, again = e.capture_and_readout(state, qs)
                assert again.tobytes() == want.tobytes()
                assert all(st_c.tensor(li, 2).tobytes() == st_a.tensor(li, 2).tobytes() for li in range(cfg.num_layers) if st_a.tensor(li, 2) is not None)
                st_c.free()
        st_a.free()
        st_b.free()
    # a request that does not fit one pass takes the two-pass order by itself
    state = rng.integers(0, vocab, 900, dtype=np.uint32)
    qs = [rng.integers(0, vocab, 100, dtype=np.uint32) for _ in range(3)]
    st_a = e.capture_state(state)
    want = e.readout_state_once_batch(st_a, qs)
    st_b, got = e.capture_and_readout(state, qs)
    assert got.tobytes() == want.tobytes()
    e.close()


@pytest.mark.parametrize("precision", [0, 3])
def test_cold_request_same_bits_with_flushed_caches(dcd, precision):
    """A cold request repeated with every cache line evicted in between (different arrival times of every tile, the state's delta
    rule on its own stream): logits and cache tensors identical run after run, one-pass equal to capture + question pass; the
    second case has so few question rows that the attention splits its key range over CTAs."""
    import torch
    cfg = dcd.d3_config(num_layers=4, dtype=1, vocab=4096)
    opt = dcd.Options()
    opt.max_pass_tokens = 6144
    opt.precision = precision
    e = dcd.Engine(cfg, opt)
    e.init_random(0)
    rng = np.random.Generator(np.random.PCG64(21))
    flush = torch.empty(300 << 20, dtype=torch.uint8, device="cuda")
    for S, lens in ((1100, rng.integers(16, 161, 12)), (4096, [16, 20])):
        state = rng.integers(0, 4096, S, dtype=np.uint32)
        qs = [rng.integers(0, 4096, int(n), dtype=np.uint32) for n in lens]
        first = None
        for _ in range(5):
            flush.random_(0, 256)
            torch.cuda.synchronize()
            st, out = e.capture_and_readout(state, qs)
            sig = [st.tensor(li, k).tobytes() for li in range(cfg.num_layers) for k in range(4) if st.tensor(li, k) is not None]
            st.free()
            if first is None:
                first = (out.tobytes(), sig)
            else:
                assert out.tobytes() == first[0] and sig == first[1]
        st = e.capture_state(state)
        two = e.readout_state_once_batch(st, qs)
        st.free()
        assert two.tobytes() == first[0]
    e.close()

