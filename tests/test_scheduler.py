"""CPU tests of the request scheduler against a fake engine (no GPU).

The scheduler is the C++ twin of the reference's BatchHandle (src/batch.rs). The fake engine implements the
operation table in Python: it records every call, computes answers from a closed formula, keeps a byte ledger for
mem_info, and fails on request with host-made errors (an "out of memory" text, a refused restore). Nothing here
touches a device. Ordering is made deterministic by parking the worker inside a first "plug" request while the
requests under test are queued."""
import ctypes as C
import threading

import numpy as np
import pytest

MIB = 1 << 20
ROWS = 5


class FakeEngine:
    def __init__(self, dcd, total=64 * 1024 * MIB, state_bytes=lambda n: n * MIB, reserve=lambda n: 100 * MIB):
        from decidra_b200 import _lib
        self.lib = _lib
        self.total, self.used, self.pooled = total, 0, 0
        self.state_bytes, self.reserve = state_bytes, reserve
        self.dev, self.host = {}, {}       # handle -> tokens
        self.next = 1
        self.log = []
        self.fail = {}                     # op -> list of messages to fail with (popped per call)
        self.errbuf = C.create_string_buffer(512)
        self.fail_capture_of = None        # (state tokens, message): the capture of that state always fails
        self.gate = None                   # (state tuple, threading.Event): capture of that state waits for the event
        self.entered = threading.Event()
        ops = _lib.SchedEngineOps()
        ops.ctx = None
        ops.readout_rows = ROWS
        self._cbs = dict(
            rebind_blas=_lib.OP_INT_CTX(lambda ctx: self._log("rebind") or 0),
            capture_state=_lib.OP_CAPTURE(self._capture), readout=_lib.OP_READOUT(self._readout),
            offload=_lib.OP_MOVE(self._offload), restore=_lib.OP_MOVE(self._restore),
            state_free=_lib.OP_FREE(self._state_free), host_free=_lib.OP_FREE(self._host_free),
            trim_pools=_lib.OP_INT_CTX(self._trim), mem_info=_lib.OP_MEM(self._mem), last_error=_lib.OP_ERR(lambda ctx: C.addressof(self.errbuf)),
            state_bytes_for=_lib.OP_SIZE(lambda ctx, n: self.state_bytes(n)), pass_reserve=_lib.OP_SIZE(lambda ctx, n: self.reserve(n)),
            readout_multi=_lib.OP_READOUT_MULTI(self._readout_multi), capture_readout=_lib.OP_CAPTURE_READOUT(self._capture_readout))
        for k, v in self._cbs.items():
            setattr(ops, k, v)
        self.ops = ops

    def _log(self, *what):
        self.log.append(what)

    def _failing(self, op):
        q = self.fail.get(op)
        if q:
            self.errbuf.value = q.pop(0).encode()
            return True
        return False

    def _capture(self, ctx, ids, n, out):
        tokens = tuple(ids[i] for i in range(n))
        if self.gate and self.gate[0] == tokens:
            self.entered.set()
            assert self.gate[1].wait(20)
        self._log("capture", tokens)
        if self.fail_capture_of is not None and tokens == tuple(self.fail_capture_of[0]):
            self.errbuf.value = self.fail_capture_of[1].encode()
            return 4
        if self._failing("capture"):
            return 2
        h = self.next
        self.next += 1
        self.dev[h] = tokens
        self.used += self.state_bytes(n)
        out[0] = h
        return 0

    @staticmethod
    def answer(state, question):
        s, q = sum(state) % 97, sum(question) % 89
        return np.array([s + q * (j + 1) + 0.25 * len(question) for j in range(ROWS)], dtype=np.float32)

    def _readout(self, ctx, st, qs, lens, B, out):
        questions = [tuple(qs[i][k] for k in range(lens[i])) for i in range(B)]
        self._log("readout", self.dev[st], tuple(questions))
        if self._failing("readout"):
            return 2
        for i, q in enumerate(questions):
            a = self.answer(self.dev[st], q)
            for j in range(ROWS):
                out[i * ROWS + j] = a[j]
        return 0

    def _readout_multi(self, ctx, states, n_states, qs, lens, state_of, B, out):
        toks = [self.dev[states[k]] for k in range(n_states)]
        questions = [tuple(qs[i][k] for k in range(lens[i])) for i in range(B)]
        sof = tuple(state_of[i] for i in range(B))
        self._log("readout_multi", tuple(toks), tuple(questions), sof)
        if self._failing("readout_multi"):
            return 1
        for i, q in enumerate(questions):
            a = self.answer(toks[sof[i]], q)
            for j in range(ROWS):
                out[i * ROWS + j] = a[j]
        return 0

    def _capture_readout(self, ctx, ids, n, qs, lens, B, st_out, out):
        tokens = tuple(ids[i] for i in range(n))
        questions = [tuple(qs[i][k] for k in range(lens[i])) for i in range(B)]
        self._log("capture_readout", tokens, tuple(questions))
        if self._failing("capture_readout"):
            return 2
        h = self.next
        self.next += 1
        self.dev[h] = tokens
        self.used += self.state_bytes(n)
        st_out[0] = h
        for i, q in enumerate(questions):
            a = self.answer(tokens, q)
            for j in range(ROWS):
                out[i * ROWS + j] = a[j]
        return 0

    def _offload(self, ctx, st, out):
        self._log("offload", self.dev[st])
        if self._failing("offload"):
            return 2
        h = self.next
        self.next += 1
        self.host[h] = self.dev[st]
        out[0] = h
        return 0

    def _restore(self, ctx, hs, out):
        self._log("restore", self.host[hs])
        if self._failing("restore"):
            return 4
        h = self.next
        self.next += 1
        self.dev[h] = self.host[hs]
        self.used += self.state_bytes(len(self.host[hs]))
        out[0] = h
        return 0

    def _state_free(self, ctx, st):
        tokens = self.dev.pop(st)
        self._log("state_free", tokens)
        b = self.state_bytes(len(tokens))
        self.used -= b
        self.pooled += b                   # freed blocks stay in the pool until a trim

    def _host_free(self, ctx, hs):
        self._log("host_free", self.host.pop(hs))

    def _trim(self, ctx):
        self._log("trim")
        self.pooled = 0
        return 0

    def _mem(self, ctx, free, total):
        free[0] = self.total - self.used - self.pooled
        total[0] = self.total
        return 0

    def calls(self, op):
        return [c for c in self.log if c[0] == op]


@pytest.fixture
def mk(dcd):
    from decidra_b200 import scheduler
    made = []

    def make(fake=None, **opt):
        fake = fake or FakeEngine(dcd)
        defaults = dict(batch_window_us=20000, state_cache_bytes=1 << 40, host_state_cache_bytes=1 << 40)
        defaults.update(opt)
        h = scheduler.BatchHandle(ops=fake.ops, **defaults)
        made.append(h)
        return h, fake

    yield make
    for h in made:
        h.close()


PLUG = (9, 9, 9)


def plug(h, fake):
    """Park the worker inside the capture of a first request; returns (ticket, release event)."""
    ev = threading.Event()
    fake.gate = (PLUG, ev)
    fake.entered.clear()
    t = h.submit_state_once(PLUG, [[1]])
    assert fake.entered.wait(20)
    return t, ev


def test_miss_then_gpu_hit_and_answers(mk):
    h, fake = mk()
    A = [3, 1, 4, 1, 5]
    qs = [[2, 7], [1, 8, 2, 8]]
    got = h.submit_state_once(A, qs).result()
    assert np.array_equal(got, np.stack([fake.answer(A, q) for q in qs]))
    s = h.stats()
    assert (s["requests_miss"], s["captures"], s["state_tokens"], s["questions_answered"], s["question_tokens"]) == (1, 1, 5, 2, 6)
    assert (s["gpu_entries"], s["gpu_bytes"], s["groups_success"], s["worker_alive"]) == (1, 5 * MIB, 1, 1)
    got2 = h.submit_state_once(A, [[5]]).result()
    assert np.array_equal(got2[0], fake.answer(A, [5]))
    s = h.stats()
    assert (s["requests_gpu_hit"], s["captures"], s["reused_tokens"]) == (1, 1, 5)
    assert len(fake.calls("capture")) == 1 and fake.log[0] == ("rebind",)
    assert (s["waiting"], s["running"], s["channel"]) == (0, 0, 0)


def test_coalescing_groups_by_exact_state_in_first_seen_order(mk):
    h, fake = mk(batch_requests=8, batch_rows=64)
    pt, ev = plug(h, fake)
    A, B = [1, 2, 3], [1, 2, 4]
    t1 = h.submit_state_once(A, [[10], [11, 12]])
    t2 = h.submit_state_once(B, [[20]])
    t3 = h.submit_state_once(A, [[30]])
    t4 = h.submit_state_once(A, [[40]], digest=b"\x01" * 32)     # same tokens, different media digest: another state
    ev.set()
    pt.result()
    r1, r2, r3, r4 = t1.result(), t2.result(), t3.result(), t4.result()
    reads = fake.calls("readout")[1:]
    assert reads == [("readout", tuple(A), ((10,), (11, 12), (30,))), ("readout", tuple(B), ((20,),)), ("readout", tuple(A), ((40,),))]
    assert np.array_equal(r1, np.stack([fake.answer(A, [10]), fake.answer(A, [11, 12])]))
    assert np.array_equal(r3[0], fake.answer(A, [30])) and np.array_equal(r2[0], fake.answer(B, [20])) and r4.shape == (1, ROWS)
    assert [c[1] for c in fake.calls("capture")] == [PLUG, tuple(A), tuple(B), tuple(A)]
    s = h.stats()
    assert s["group_requests"] == 5 and s["groups_success"] == 4 and s["requests_miss"] == 5


def test_row_budget_and_zero_window(mk):
    h, fake = mk(batch_requests=8, batch_rows=3)
    pt, ev = plug(h, fake)
    A = [7, 7]
    ts = [h.submit_state_once(A, [[i], [i + 1]]) for i in (1, 3, 5)]
    ev.set()
    for t in ts:
        t.result()
    # rows are the SUM of questions in the group: 2, then 4 >= 3 closes the pass; the third request runs alone
    reads = [c[2] for c in fake.calls("readout")[1:]]
    assert reads == [((1,), (2,), (3,), (4,)), ((5,), (6,))]
    h2, fake2 = mk(batch_requests=8, batch_rows=64, batch_window_us=0)
    pt, ev = plug(h2, fake2)
    ts = [h2.submit_state_once(A, [[i]]) for i in (1, 2, 3)]
    ev.set()
    for t in ts:
        t.result()
    assert [c[2] for c in fake2.calls("readout")[1:]] == [((1,),), ((2,),), ((3,),)]   # a zero window never coalesces


def test_full_device_tier_spills_to_host_and_restores(mk):
    h, fake = mk(state_cache_entries=2)
    A, B, Cc = [1] * 4, [2] * 4, [3] * 4
    for st in (A, B, Cc):
        h.submit_state_once(st, [[1]]).result()
    s = h.stats()
    assert (s["gpu_entries"], s["host_entries"], s["offloads"], s["offload_bytes"]) == (2, 1, 1, 4 * MIB)
    assert fake.calls("offload") == [("offload", tuple(Cc))] and ("state_free", tuple(Cc)) in fake.log
    got = h.submit_state_once(Cc, [[6, 6]]).result()
    assert np.array_equal(got[0], fake.answer(Cc, [6, 6]))
    s = h.stats()
    assert (s["requests_host_hit"], s["restores"], s["restore_bytes"], s["captures"]) == (1, 1, 4 * MIB, 3)
    assert (s["gpu_entries"], s["host_entries"]) == (2, 1)       # still no room on the device: the host copy stays
    assert fake.calls("restore") == [("restore", tuple(Cc))]


def test_host_budget_evicts_oldest(mk):
    h, fake = mk(state_cache_entries=1, host_state_cache_bytes=9 * MIB)
    states = [[i] * 4 for i in (1, 2, 3, 4)]                   # 4 MiB each; the device tier holds one
    for st in states:
        h.submit_state_once(st, [[1]]).result()
    s = h.stats()
    assert (s["gpu_entries"], s["host_entries"], s["host_bytes"], s["evict_host_budget"]) == (1, 2, 8 * MIB, 1)
    assert fake.calls("host_free") == [("host_free", tuple(states[1]))]


def test_unpinned_cache_evicts_for_the_byte_budget(mk):
    h, fake = mk(state_cache_entries=4, state_cache_bytes=10 * MIB, pin_cache=0)
    A, B, Cc = [1] * 4, [2] * 4, [3] * 4
    for st in (A, B, Cc):
        h.submit_state_once(st, [[1]]).result()
    s = h.stats()
    assert (s["evict_gpu_byte_limit"], s["gpu_entries"], s["host_entries"]) == (1, 2, 0)
    h.submit_state_once(B, [[1]]).result()                       # B survived, A was the oldest
    assert h.stats()["requests_gpu_hit"] == 1 and [c[1] for c in fake.calls("capture")] == [tuple(A), tuple(B), tuple(Cc)]


def test_headroom_trims_then_offloads_then_fails(dcd, mk):
    fake = FakeEngine(dcd, total=400 * MIB, state_bytes=lambda n: n * 10 * MIB, reserve=lambda n: 200 * MIB)
    h, _ = mk(fake)
    A, B = [1] * 10, [2] * 10                                    # 100 MiB each
    h.submit_state_once(A, [[1]]).result()                       # free 400 -> needs 300: fine; A cached (100 used)
    assert fake.calls("trim") == [] and fake.calls("offload") == []
    h.submit_state_once(B, [[1]]).result()                       # free 300, needs 300: fine
    # both cached: 200 used. A third state needs 300 free: trim (nothing pooled), then the oldest entry goes to the host
    Cc = [3] * 10
    h.submit_state_once(Cc, [[1]]).result()
    assert fake.calls("offload")[0] == ("offload", tuple(A)) and len(fake.calls("trim")) >= 2
    s = h.stats()
    assert s["offloads"] >= 1 and s["fail_headroom"] == 0
    # a state that cannot fit even with every entry offloaded fails with the reference's text
    big = [4] * 25                                               # 250 + 200 MiB > 400 MiB
    t = h.submit_state_once(big, [[1], [2]])
    with pytest.raises(dcd.EngineError, match=r"insufficient GPU memory for state capture/restore: \d+ MiB free, 450 MiB required") as ei:
        t.result()
    assert ei.value.code == 7
    s = h.stats()
    assert (s["fail_headroom"], s["questions_failed"], s["groups_failed"], s["gpu_entries"]) == (1, 2, 1, 0)


def test_out_of_memory_is_retried_once_per_phase(mk):
    h, fake = mk()
    fake.fail["capture"] = ["capture_state: CUDA out of memory"]
    got = h.submit_state_once([1, 2], [[3]]).result()
    assert np.array_equal(got[0], fake.answer([1, 2], [3]))
    s = h.stats()
    assert (s["oom_retry_capture"], s["captures"], s["fail_state_capture"]) == (1, 1, 0) and len(fake.calls("capture")) == 2
    fake.fail["readout"] = ["question pass: CUDA out of memory"]
    h.submit_state_once([1, 2], [[4]]).result()
    assert h.stats()["oom_retry_question"] == 1
    # two failures in a row: the second is final
    fake.fail["capture"] = ["x: CUDA out of memory", "y: CUDA out of memory"]
    with pytest.raises(Exception, match="state capture failed: y: CUDA out of memory"):
        h.submit_state_once([5, 5], [[1]]).result()
    # any other error is not retried
    fake.fail["readout"] = ["token 99999 is outside the vocabulary"]
    n = len(fake.calls("readout"))
    with pytest.raises(Exception, match="state-once question pass failed: token 99999"):
        h.submit_state_once([1, 2], [[1]]).result()
    s = h.stats()
    assert len(fake.calls("readout")) == n + 1 and (s["fail_state_capture"], s["fail_question_pass"], s["oom_retry_question"]) == (1, 1, 1)
    # the failed question pass dropped the state it had taken out of the cache
    assert s["gpu_entries"] == 0


def test_restore_failure_keeps_the_host_copy(mk):
    h, fake = mk(state_cache_entries=1)
    A, B = [1] * 3, [2] * 3
    h.submit_state_once(A, [[1]]).result()
    h.submit_state_once(B, [[1]]).result()                       # B spills to the host tier
    fake.fail["restore"] = ["restore: pinned copy failed"]
    with pytest.raises(Exception, match="state restore failed: restore: pinned copy failed"):
        h.submit_state_once(B, [[1]]).result()
    s = h.stats()
    assert (s["fail_state_restore"], s["host_entries"], s["requests_host_hit"]) == (1, 1, 1)
    assert np.array_equal(h.submit_state_once(B, [[2]]).result()[0], fake.answer(B, [2]))


def test_cancelled_request_is_skipped(mk):
    h, fake = mk()
    pt, ev = plug(h, fake)
    X = [8, 8, 8, 8]
    t = h.submit_state_once(X, [[1], [2], [3]])
    keep = h.submit_state_once([5], [[1]])
    t.cancel()
    ev.set()
    pt.result()
    keep.result()
    with pytest.raises(Exception, match="cancelled"):
        t.result()
    s = h.stats()
    assert (s["cancelled_queued"], s["questions_cancelled"]) == (1, 3)
    assert tuple(X) not in [c[1] for c in fake.calls("capture")]


def test_queue_full_and_option_checks(dcd, mk):
    from decidra_b200 import scheduler
    h, fake = mk(max_queue=2, submit_timeout_us=2000)
    pt, ev = plug(h, fake)                                       # slot 1 (running)
    t2 = h.submit_state_once([1], [[1]])                         # slot 2 (queued)
    with pytest.raises(dcd.EngineError, match="d3-turbo queue is full; retry shortly") as ei:
        h.submit_state_once([2], [[1]])
    assert ei.value.code == 6 and h.stats()["reject_queue_full"] == 1
    ev.set()
    pt.result(); t2.result()
    h.submit_state_once([2], [[1]]).result()                     # slots are free again
    for bad, text in ((dict(max_queue=0), "max_queue"), (dict(batch_requests=0), "batch_requests"), (dict(batch_rows=0), "batch_rows"),
                      (dict(batch_window_us=50001), "at most 50000")):
        with pytest.raises(dcd.EngineError, match=text):
            scheduler.BatchHandle(ops=fake.ops, **bad)
    d = scheduler.default_options()
    assert (d.max_queue, d.batch_requests, d.batch_rows, d.batch_window_us, d.state_cache_entries) == (64, 32, 32, 2000, 16)
    assert (d.state_cache_bytes, d.host_state_cache_bytes, d.pin_cache, d.sched_priority) == (5 << 30, 8 << 30, 1, 0)


def test_priority_runs_the_cheapest_group_first(mk):
    h, fake = mk(sched_priority=1, batch_requests=8, batch_rows=64)
    h.submit_state_once([6] * 50, [[1]]).result()                # a long state that is already cached costs nothing
    pt, ev = plug(h, fake)
    long_new = h.submit_state_once([7] * 40, [[1]])              # cost 40 + 1
    long_cached = h.submit_state_once([6] * 50, [[1, 2, 3]])     # cost 0 + 3
    short_new = h.submit_state_once([8] * 5, [[1, 2]])           # cost 5 + 2
    ev.set()
    for t in (pt, long_new, long_cached, short_new):
        t.result()
    order = [c[1][0] for c in fake.calls("readout")[2:]]
    assert order == [6, 8, 7]


def test_close_finishes_queued_requests(mk):
    h, fake = mk()
    pt, ev = plug(h, fake)
    ts = [h.submit_state_once([i], [[i]]) for i in (1, 2, 3)]
    closer = threading.Thread(target=h.close)
    closer.start()
    ev.set()
    closer.join(20)
    assert not closer.is_alive()
    for i, t in zip((1, 2, 3), ts):
        assert np.array_equal(t.result()[0], fake.answer([i], [i]))
    # both tiers were released
    assert fake.dev == {} and fake.host == {}


def test_cross_state_pass_serves_several_groups_at_once(mk):
    h, fake = mk(cross_state_pass=1, batch_requests=8, batch_rows=64)
    pt, ev = plug(h, fake)
    A, B = [1, 2, 3], [4, 5]
    t1 = h.submit_state_once(A, [[10], [11, 12]])
    t2 = h.submit_state_once(B, [[20]])
    t3 = h.submit_state_once(A, [[30]])
    ev.set()
    pt.result()
    r1, r2, r3 = t1.result(), t2.result(), t3.result()
    multi = fake.calls("readout_multi")
    assert multi == [("readout_multi", (tuple(A), tuple(B)), ((10,), (11, 12), (30,), (20,)), (0, 0, 0, 1))]
    assert len(fake.calls("readout")) == 1                       # the plug's own pass only
    assert np.array_equal(r1, np.stack([fake.answer(A, [10]), fake.answer(A, [11, 12])]))
    assert np.array_equal(r2[0], fake.answer(B, [20])) and np.array_equal(r3[0], fake.answer(A, [30]))
    s = h.stats()
    assert (s["cross_state_passes"], s["requests_fallback"], s["captures"], s["groups_success"], s["questions_answered"]) == (1, 0, 3, 3, 5)
    assert (s["gpu_entries"], s["waiting"], s["running"]) == (3, 0, 0)
    # both states went back to the device tier; a batch with a single group takes the ordinary pass
    assert np.array_equal(h.submit_state_once(B, [[7]]).result()[0], fake.answer(B, [7]))
    s = h.stats()
    assert s["requests_gpu_hit"] == 1 and s["cross_state_passes"] == 1 and len(fake.calls("readout")) == 2


def test_cross_state_pass_falls_back_and_isolates_failures(mk):
    h, fake = mk(cross_state_pass=1, batch_requests=8, batch_rows=64)
    pt, ev = plug(h, fake)
    A, B, Cc = [1, 1], [2, 2], [3, 3]
    fake.fail["readout_multi"] = ["pass of 99999 tokens exceeds max_pass_tokens: split the call"]
    ta, tb = h.submit_state_once(A, [[1]]), h.submit_state_once(B, [[2], [3]])
    ev.set()
    pt.result()
    assert np.array_equal(ta.result()[0], fake.answer(A, [1])) and np.array_equal(tb.result()[1], fake.answer(B, [3]))
    s = h.stats()
    assert (s["cross_state_passes"], s["requests_fallback"], s["groups_success"], s["captures"]) == (0, 2, 3, 3)
    assert [c[1] for c in fake.calls("readout")[1:]] == [tuple(A), tuple(B)]   # one pass per group, states captured once
    # a group whose state cannot be captured fails alone; the other two still share a pass
    pt, ev = plug2(h, fake)
    fake.fail_capture_of = (Cc, "capture: device lost its mind")
    tc_ = h.submit_state_once(Cc, [[9]])
    ta, tb = h.submit_state_once(A, [[4]]), h.submit_state_once(B, [[5]])
    ev.set()
    pt.result()
    with pytest.raises(Exception, match="state capture failed: capture: device lost its mind"):
        tc_.result()
    assert np.array_equal(ta.result()[0], fake.answer(A, [4])) and np.array_equal(tb.result()[0], fake.answer(B, [5]))
    s = h.stats()
    assert (s["cross_state_passes"], s["fail_state_capture"], s["groups_failed"]) == (1, 1, 1)
    assert fake.calls("readout_multi")[-1][3] == (0, 1)


def plug2(h, fake):
    """A second plug on a scheduler whose first plug state is already cached: use a fresh state."""
    ev = threading.Event()
    fake.gate = ((8, 8, 8, 8), ev)
    fake.entered.clear()
    t = h.submit_state_once((8, 8, 8, 8), [[1]])
    assert fake.entered.wait(20)
    return t, ev


@pytest.mark.parametrize("cross", [0, 1])
def test_cross_state_pass_under_memory_pressure_answers_like_the_sequential_order(dcd, mk, cross):
    """Three 250 MiB states on a 700 MiB device, 100 MiB reserved per pass. One group at a time, the third capture offloads the
    oldest cached state and succeeds. With cross_state_pass the first two states are in hand (not in the device tier, so nothing
    can offload them) when the third does not fit: the scheduler serves and releases the two it holds, then acquires the third
    alone. Both modes answer every request."""
    fake = FakeEngine(dcd, total=700 * MIB)
    h, fake = mk(fake, cross_state_pass=cross, batch_requests=8, batch_rows=64)
    pt, ev = plug(h, fake)
    A, B, Cc = [1] * 250, [2] * 250, [3] * 250
    ta, tb, tc_ = h.submit_state_once(A, [[1], [2]]), h.submit_state_once(B, [[3]]), h.submit_state_once(Cc, [[4], [5]])
    ev.set()
    pt.result()
    ra, rb, rc = ta.result(), tb.result(), tc_.result()
    assert np.array_equal(ra, np.stack([fake.answer(A, [1]), fake.answer(A, [2])]))
    assert np.array_equal(rb[0], fake.answer(B, [3]))
    assert np.array_equal(rc, np.stack([fake.answer(Cc, [4]), fake.answer(Cc, [5])]))
    s = h.stats()
    assert (s["groups_failed"], s["fail_headroom"], s["fail_state_capture"], s["questions_failed"]) == (0, 0, 0, 0)
    assert s["captures"] == 4 and s["offloads"] >= 1 and s["requests_miss"] == 4
    assert s["cross_state_passes"] == (1 if cross else 0)
    if cross:
        assert fake.calls("readout_multi")[0][1] == (tuple(A), tuple(B))
        assert fake.calls("readout")[-1][1] == tuple(Cc)


def test_cold_one_pass_serves_a_miss_with_one_engine_call(mk):
    """cold_one_pass = 1: a miss is one capture_readout call (state kept in the cache as after a capture); a hit is a plain readout;
    a memory failure is retried once; any other failure of the one-pass call sends the group through capture + readout, so the
    failure texts stay the reference's."""
    h, fake = mk(cold_one_pass=1)
    A, qs = [3, 1, 4], [[2, 7], [1, 8]]
    got = h.submit_state_once(A, qs).result()
    assert np.array_equal(got, np.stack([fake.answer(A, q) for q in qs]))
    assert len(fake.calls("capture_readout")) == 1 and not fake.calls("capture") and not fake.calls("readout")
    s = h.stats()
    assert (s["requests_miss"], s["captures"], s["state_tokens"], s["questions_answered"], s["question_tokens"], s["gpu_entries"]) == (1, 1, 3, 2, 4, 1)
    # the state is cached: the next request is a hit served by a plain readout
    assert np.array_equal(h.submit_state_once(A, [[5]]).result()[0], fake.answer(A, [5]))
    assert len(fake.calls("capture_readout")) == 1 and len(fake.calls("readout")) == 1
    # a memory failure: trimmed and retried once, same call
    fake.fail["capture_readout"] = ["CUDA error: out of memory"]
    B = [9, 9, 1]
    assert np.array_equal(h.submit_state_once(B, [[4]]).result()[0], fake.answer(B, [4]))
    assert len(fake.calls("capture_readout")) == 3 and h.stats()["oom_retry_capture"] == 1
    # another failure: the two steps, and their messages
    fake.fail["capture_readout"] = ["token id out of range"]
    fake.fail["readout"] = ["token id out of range"]
    with pytest.raises(Exception, match="state-once question pass failed: token id out of range"):
        h.submit_state_once([7, 7, 7], [[1]]).result()
    assert fake.calls("capture")[-1] == ("capture", (7, 7, 7))
    # and with the option off nothing changes
    h2, fake2 = mk()
    h2.submit_state_once(A, qs).result()
    assert not fake2.calls("capture_readout") and len(fake2.calls("capture")) == 1
