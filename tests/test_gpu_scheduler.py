"""The request scheduler over the real engine on the GPU: replies must be bit-identical to direct engine calls
whatever route the state took (fresh capture, device-tier hit, host-tier restore, coalesced with other requests)."""
import threading

import numpy as np
import pytest

from conftest import tiny_inputs

pytestmark = pytest.mark.gpu


def _engine(dcd):
    o = dcd.Options()
    o.max_pass_tokens = 512
    e = dcd.Engine(dcd.tiny_config(1), o)
    e.init_random(0)
    return e


def _cases(n_states=3):
    out = []
    for s in range(n_states):
        state, questions = tiny_inputs(seed=10 + s, state_len=96 + 16 * s, qlens=(12, 20, 7, 31))
        out.append((state, questions))
    return out


def test_scheduler_replies_equal_direct_calls(dcd):
    from decidra_b200 import scheduler
    e = _engine(dcd)
    cases = _cases()
    want = [e.readout_state_once_batch(e.capture_state(st), qs) for st, qs in cases]
    h = scheduler.BatchHandle(e, batch_window_us=0, state_cache_entries=1)
    # miss -> captured and kept on the device
    assert h.submit_state_once(*cases[0]).result().tobytes() == want[0].tobytes()
    # the cache's byte ledger holds what the state really takes in this engine (its config and storage type), not the
    # reference's 64 KiB per token
    st0 = e.capture_state(cases[0][0])
    assert h.stats()["gpu_bytes"] == st0.nbytes > 0 and st0.nbytes != len(cases[0][0]) * 65536
    st0.free()
    # device hit with a subset of the questions
    got = h.submit_state_once(cases[0][0], cases[0][1][1:3]).result()
    assert got.tobytes() == want[0][1:3].tobytes()
    # the device tier holds one entry: the next state spills to pinned host memory, then comes back from there
    assert h.submit_state_once(*cases[1]).result().tobytes() == want[1].tobytes()
    assert h.submit_state_once(*cases[1]).result().tobytes() == want[1].tobytes()
    s = h.stats()
    assert (s["requests_miss"], s["requests_gpu_hit"], s["requests_host_hit"]) == (2, 1, 1)
    assert (s["captures"], s["offloads"], s["restores"], s["gpu_entries"], s["host_entries"]) == (2, 1, 1, 1, 1)
    assert s["questions_answered"] == 4 + 2 + 4 + 4 and s["groups_failed"] == 0
    # an invalid request fails alone, with the engine's message behind the reference's prefix
    bad = [np.array([1, 2, 999999], dtype=np.uint32)]
    with pytest.raises(dcd.EngineError, match="state-once question pass failed"):
        h.submit_state_once(cases[0][0], bad).result()
    assert h.submit_state_once(*cases[2]).result().tobytes() == want[2].tobytes()
    h.close()
    e.close()


def test_scheduler_concurrent_clients_coalesce(dcd):
    from decidra_b200 import scheduler
    e = _engine(dcd)
    cases = _cases()
    want = [e.readout_state_once_batch(e.capture_state(st), qs) for st, qs in cases]
    h = scheduler.BatchHandle(e, batch_window_us=20000, batch_requests=16, batch_rows=64, state_cache_entries=4)
    results, errors = {}, []

    def client(tid):
        try:
            for rep in range(3):
                k = (tid + rep) % len(cases)
                st, qs = cases[k]
                lo = (tid + rep) % 3
                results[(tid, rep)] = (k, lo, h.submit_state_once(st, qs[lo:lo + 2]).result())
        except Exception as ex:  # noqa: BLE001
            errors.append(ex)

    threads = [threading.Thread(target=client, args=(t,)) for t in range(6)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(120)
    assert not errors, errors
    assert len(results) == 18
    for (k, lo, got) in results.values():
        assert got.tobytes() == want[k][lo:lo + 2].tobytes()
    s = h.stats()
    assert s["questions_answered"] == 36 and s["captures"] == 3
    assert s["group_requests"] == 18 and s["groups_success"] < 18      # some requests shared a pass
    h.close()
    e.close()


def test_scheduler_cross_state_pass(dcd):
    """cross_state_pass: requests for different states that wait together are answered by ONE question pass; the rows
    are still those of direct per-state calls, bit for bit."""
    from decidra_b200 import scheduler
    e = _engine(dcd)
    cases = _cases(4)
    want = [e.readout_state_once_batch(e.capture_state(st), qs) for st, qs in cases]
    h = scheduler.BatchHandle(e, batch_window_us=30000, batch_requests=16, batch_rows=64, state_cache_entries=8, cross_state_pass=1)
    first = h.submit_state_once(*cases[0])           # keeps the worker busy (capture + pass) while the others queue up
    tickets = [h.submit_state_once(st, qs) for st, qs in cases[1:]] + [h.submit_state_once(cases[1][0], cases[1][1][:2])]
    assert first.result().tobytes() == want[0].tobytes()
    for k, t in enumerate(tickets[:3]):
        assert t.result().tobytes() == want[k + 1].tobytes()
    assert tickets[3].result().tobytes() == want[1][:2].tobytes()
    s = h.stats()
    assert s["cross_state_passes"] >= 1 and s["requests_fallback"] == 0 and s["captures"] == 4 and s["questions_answered"] == 4 * 4 + 2
    # second round: every state is a device-tier hit and they still share a pass
    tickets = [h.submit_state_once(st, qs[::-1]) for st, qs in cases]
    for k, t in enumerate(tickets):
        assert t.result().tobytes() == want[k][::-1].tobytes()
    s = h.stats()
    assert s["captures"] == 4 and s["requests_gpu_hit"] >= 4
    h.close()
    e.close()


def test_cold_one_pass_through_the_scheduler_equals_direct_calls(dcd):
    """cold_one_pass = 1 on the real engine: a miss served by dcd_capture_and_readout gives the rows of capture + readout bit for bit,
    leaves the state in the device tier for the next request, and a bad question still fails with the reference's text."""
    from decidra_b200 import scheduler
    e = _engine(dcd)
    cases = _cases()
    want = [e.readout_state_once_batch(e.capture_state(st), qs) for st, qs in cases]
    h = scheduler.BatchHandle(e, batch_window_us=0, cold_one_pass=1)
    for (st, qs), w in zip(cases, want):
        assert h.submit_state_once(st, qs).result().tobytes() == w.tobytes()
    assert h.submit_state_once(cases[1][0], cases[1][1][:2]).result().tobytes() == want[1][:2].tobytes()
    s = h.stats()
    assert (s["requests_miss"], s["requests_gpu_hit"], s["captures"], s["gpu_entries"]) == (3, 1, 3, 3)
    bad = [np.array([1, 2, 999999], dtype=np.uint32)]
    fresh = np.arange(50, dtype=np.uint32)
    with pytest.raises(dcd.EngineError, match="state-once question pass failed"):
        h.submit_state_once(fresh, bad).result()
    h.close()
    e.close()
