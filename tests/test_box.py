"""CPU tests of the whole-box router over fake engines (no GPU): cache affinity, work stealing for cold states, answers."""
import threading

import numpy as np

from test_scheduler import FakeEngine


def make_box(dcd, n, **opt):
    from decidra_b200 import box, scheduler
    fakes = [FakeEngine(dcd) for _ in range(n)]
    defaults = dict(batch_window_us=0, state_cache_bytes=1 << 40, host_state_cache_bytes=1 << 40)
    defaults.update(opt)
    handles = [scheduler.BatchHandle(ops=f.ops, **defaults) for f in fakes]
    return box.BoxRunner(handles), fakes


def test_answers_and_affinity(dcd):
    b, fakes = make_box(dcd, 3)
    try:
        states = [[i, i + 1, i + 2, 7] for i in range(12)]
        first = {}
        for s in states:
            t = b.submit_state_once(s, [[1, 2], [3]])
            got = t.result()
            assert np.array_equal(got, np.stack([FakeEngine.answer(s, q) for q in ([1, 2], [3])]))
            first[tuple(s)] = t.replica
        # a state that was served goes back to the replica that holds its capture, and is not captured again
        for s in states:
            t = b.submit_state_once(s, [[5, 5]])
            assert np.array_equal(t.result()[0], FakeEngine.answer(s, [5, 5]))
            assert t.replica == first[tuple(s)] and not t.stolen
        st = b.stats()
        assert sum(st["requests"]) == 24 and sum(st["affinity_hits"]) == 12
        assert sum(len(f.calls("capture")) for f in fakes) == 12
        assert sum(s["requests_gpu_hit"] for s in st["schedulers"]) == 12
        # with nothing in flight every cold state went to its static home
        from decidra_b200 import box, replicas
        assert all(first[tuple(s)] == replicas.state_affinity_rank(box.state_key(s), 3) for s in states)
        assert sum(st["steals"]) == 0
    finally:
        b.close()


def test_cold_states_go_to_the_least_loaded_replica(dcd):
    """One replica is parked inside a capture: cold states whose home it is are taken by the others, and nothing waits for it."""
    from decidra_b200 import box, replicas
    b, fakes = make_box(dcd, 2)
    try:
        # a state whose home is replica 0, used to park replica 0's worker
        plug = next([9, 9, k] for k in range(100) if replicas.state_affinity_rank(box.state_key([9, 9, k]), 2) == 0)
        ev = threading.Event()
        fakes[0].gate = (tuple(plug), ev)
        tp = b.submit_state_once(plug, [[1]])
        assert fakes[0].entered.wait(20)
        assert tp.replica == 0 and b.in_flight() == [1, 0]
        homes0 = [[4, 4, k] for k in range(200) if replicas.state_affinity_rank(box.state_key([4, 4, k]), 2) == 0][:5]
        for s in homes0:
            t = b.submit_state_once(s, [[2]])
            assert t.replica == 1 and t.stolen          # replica 0 is busy: the cold state is stolen
            assert np.array_equal(t.result()[0], FakeEngine.answer(s, [2]))
        assert b.stats()["steals"] == [0, 5]
        # the stolen states now live on replica 1 and stay there even when replica 0 is free again
        ev.set()
        tp.result()
        assert b.in_flight() == [0, 0]
        t = b.submit_state_once(homes0[0], [[3]])
        assert t.replica == 1 and not t.stolen and np.array_equal(t.result()[0], FakeEngine.answer(homes0[0], [3]))
        assert len(fakes[1].calls("capture")) == 5 and len(fakes[0].calls("capture")) == 1
    finally:
        b.close()


def test_many_threads(dcd):
    b, fakes = make_box(dcd, 4)
    errs = []

    def client(c):
        try:
            for i in range(20):
                s = [c, i % 5, 11]
                q = [[c + 1, i + 1]]
                assert np.array_equal(b.submit_state_once(s, q).result()[0], FakeEngine.answer(s, q[0]))
        except Exception as ex:  # noqa: BLE001
            errs.append(repr(ex))

    try:
        ts = [threading.Thread(target=client, args=(c,)) for c in range(8)]
        [t.start() for t in ts]
        [t.join() for t in ts]
        assert not errs, errs
        st = b.stats()
        assert sum(st["requests"]) == 160 and b.in_flight() == [0, 0, 0, 0]
        # 40 distinct states: each was captured once, on one replica
        assert sum(len(f.calls("capture")) for f in fakes) == 40
    finally:
        b.close()
