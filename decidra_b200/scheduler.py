"""Host-side mirror of juanqui/decidra's ``BatchHandle`` (src/batch.rs:32-36, 265-427): the single
worker that owns the engine, coalesces requests, groups them by exact state and keeps captured states
in a device tier and a pinned-host second level. The scheduler itself is C++ inside
``libdecidra_b200.so`` (``csrc/scheduler.cpp``); this module marshals requests and replies.
"""
from __future__ import annotations

import ctypes as C
from typing import Sequence

import numpy as np

from . import _lib
from .engine import Engine, EngineError


def default_options() -> _lib.SchedOptions:
    """The reference's defaults (src/config.rs:16-28)."""
    o = _lib.SchedOptions()
    _lib.load().dcd_sched_default_options(C.byref(o))
    return o


class Ticket:
    """The receiver of one request's reply (``oneshot::Receiver<Result<Vec<Vec<f32>>, String>>``)."""

    def __init__(self, handle, questions: int, readout_rows: int):
        self._h, self._n, self._r = handle, questions, readout_rows

    def done(self) -> bool:
        return bool(_lib.load().dcd_ticket_done(self._h))

    def cancel(self) -> None:
        """The client went away: the request is skipped if the worker has not started it."""
        _lib.load().dcd_ticket_cancel(self._h)

    def result(self) -> np.ndarray:
        """Block for the reply: [questions, readout_rows] f32, or raise with the worker's failure text."""
        lib = _lib.load()
        out = np.empty((self._n, self._r), dtype=np.float32)
        rc = lib.dcd_ticket_wait(self._h, out.ctypes.data_as(_lib.FP), out.size)
        if rc:
            raise EngineError(rc, (lib.dcd_ticket_error(self._h) or b"").decode())
        return out

    def free(self):
        if self._h:
            _lib.load().dcd_ticket_free(self._h)
            self._h = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class BatchHandle:
    """``BatchHandle::spawn``: after this call the worker thread is the only user of ``engine``."""

    def __init__(self, engine: Engine | None = None, options: _lib.SchedOptions | None = None, *, ops: _lib.SchedEngineOps | None = None,
                 **overrides):
        self._h = None
        lib = _lib.load()
        o = options or default_options()
        for k, v in overrides.items():
            setattr(o, k, v)
        self.options = o
        out = C.c_void_p()
        if ops is not None:
            self._keep = ops  # the callbacks must outlive the worker
            self.readout_rows = int(ops.readout_rows)
            rc = lib.dcd_scheduler_create_with_ops(C.byref(ops), C.byref(o), C.byref(out))
        else:
            self._keep = engine
            self.readout_rows = int(engine.cfg.readout_rows)
            rc = lib.dcd_scheduler_create(engine._h, C.byref(o), C.byref(out))
        if rc:
            raise EngineError(rc, (lib.dcd_scheduler_last_error() or b"").decode())
        self._h = out

    @classmethod
    def spawn(cls, engine: Engine, max_queue: int, batch_requests: int, batch_rows: int, batch_window_us: int, state_cache_entries: int,
              state_cache_bytes: int, host_state_cache_bytes: int) -> "BatchHandle":
        """Same argument list as the reference's ``BatchHandle::spawn``."""
        return cls(engine, max_queue=max_queue, batch_requests=batch_requests, batch_rows=batch_rows, batch_window_us=batch_window_us,
                   state_cache_entries=state_cache_entries, state_cache_bytes=state_cache_bytes,
                   host_state_cache_bytes=host_state_cache_bytes)

    def submit_state_once(self, state: Sequence[int], questions: Sequence[Sequence[int]], digest: bytes | None = None) -> Ticket:
        """``submit_state_once``: returns at once; ``Ticket.result()`` resolves when the worker has finished the
        request's question batch. Raises EngineError(E_OVERLOADED) when the queue is full."""
        lib = _lib.load()
        st = np.ascontiguousarray(state, dtype=np.uint32)
        arrs = [np.ascontiguousarray(q, dtype=np.uint32) for q in questions]
        B = len(arrs)
        ptrs = (_lib.U32P * max(B, 1))(*[a.ctypes.data_as(_lib.U32P) for a in arrs])
        lens = (C.c_size_t * max(B, 1))(*[a.size for a in arrs])
        if digest is not None and len(digest) != 32:
            raise ValueError("digest must be 32 bytes")
        out = C.c_void_p()
        rc = lib.dcd_scheduler_submit(self._h, st.ctypes.data_as(_lib.U32P), st.size, ptrs, lens, B, digest, C.byref(out))
        if rc:
            raise EngineError(rc, (lib.dcd_scheduler_last_error() or b"").decode())
        return Ticket(out, B, self.readout_rows)

    def stats(self) -> dict:
        s = _lib.SchedStats()
        _lib.load().dcd_scheduler_stats(self._h, C.byref(s))
        return {n: int(getattr(s, n)) for n in _lib.SCHED_STAT_NAMES}

    def close(self):
        """Close the queue, let the worker finish what was queued, free both cache tiers, join the thread."""
        if self._h:
            _lib.load().dcd_scheduler_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
