"""The whole-box router over real engines (two replicas on the one GPU of the test box): answers equal the engine's own,
a served state returns to its replica without a second capture, a busy replica's cold states are taken by the other."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_box_of_two_replicas_answers_like_one_engine(dcd):
    from decidra_b200 import box, scheduler
    cfg = dcd.tiny_config(dtype=1)
    engines = []
    for _ in range(3):
        opt = dcd.Options()
        opt.max_pass_tokens = 1024
        e = dcd.Engine(cfg, opt, device=0)
        e.init_random(0)
        engines.append(e)
    direct = engines[2]
    b = box.BoxRunner([scheduler.BatchHandle(e, batch_window_us=0) for e in engines[:2]])
    try:
        rng = np.random.Generator(np.random.PCG64(5))
        states = [rng.integers(0, cfg.vocab, int(n), dtype=np.uint32) for n in rng.integers(40, 200, 10)]
        qsets = [[rng.integers(0, cfg.vocab, int(n), dtype=np.uint32) for n in rng.integers(5, 40, 3)] for _ in states]
        tickets = [b.submit_state_once(s, q) for s, q in zip(states, qsets)]   # all in flight at once: both replicas get work
        got = [t.result() for t in tickets]
        where = [t.replica for t in tickets]
        assert set(where) == {0, 1}
        for s, q, g in zip(states, qsets, got):
            st = direct.capture_state(s)
            want = direct.readout_state_once_batch(st, q)
            st.free()
            assert np.array_equal(g, want)
        # warm: back to the same replica, no new capture
        again = [b.submit_state_once(s, q[:1]) for s, q in zip(states, qsets)]
        for t, w, g in zip(again, where, got):
            assert np.array_equal(t.result()[0], g[0]) and t.replica == w
        st = b.stats()
        assert sum(st["affinity_hits"]) == 10 and sum(x["captures"] for x in st["schedulers"]) == 10
        assert sum(x["requests_gpu_hit"] for x in st["schedulers"]) == 10
    finally:
        b.close()
        for e in engines:
            e.close()
