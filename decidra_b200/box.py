"""Whole-box serving: one process, one engine and one request scheduler per GPU, one router in front of them.

The reference serves one GPU per process (``BatchHandle`` owns the only engine, src/batch.rs:265-427 in juanqui/decidra) and is
scaled by running replicas behind a load balancer. Every question attends only to its own state's cache and the reference's
cache key is exactly (state ids, image digest) (src/batch.rs:506-513), so a state and all its questions belong to one replica
and nothing crosses GPUs on the data path: no collective, no peer access. What a box-level front end has to decide is only
where a state goes:

* a state that a replica already served goes back to it: its capture sits in that replica's state cache (cache affinity);
* a state nobody has seen has no cache to be near, so it goes to the replica with the fewest requests in flight, and on a
  tie to its static home ``replicas.state_affinity_rank``: a GPU that runs faster, or that drew shorter states, empties
  its queue sooner and takes more of the cold states (work stealing), instead of every step waiting for the slowest rank.

Each replica keeps its own ``scheduler.BatchHandle`` (coalescing window, exact-state grouping, two-tier state cache), so a
request's life inside a replica is the reference's. The router holds no device memory and touches no CUDA call.
"""
from __future__ import annotations

import hashlib
import threading
from collections import OrderedDict
from typing import Sequence

import numpy as np

from .replicas import state_affinity_rank
from .scheduler import BatchHandle, Ticket


def state_key(state: Sequence[int], digest: bytes | None = None) -> bytes:
    """The reference's cache key: the state's token ids and the image digest (src/batch.rs:506-513)."""
    h = hashlib.blake2b(np.ascontiguousarray(state, dtype=np.uint32).tobytes(), digest_size=16)
    if digest:
        h.update(digest)
    return h.digest()


class BoxTicket:
    """The reply of one routed request; ``replica`` is where it ran, ``stolen`` whether that was not its static home."""

    def __init__(self, box: "BoxRunner", ticket: Ticket, replica: int, stolen: bool):
        self._box, self._t, self.replica, self.stolen = box, ticket, replica, stolen
        self._settled = False

    def done(self) -> bool:
        return self._t.done()

    def result(self) -> np.ndarray:
        try:
            return self._t.result()
        finally:
            self._settle()

    def cancel(self) -> None:
        self._t.cancel()

    def _settle(self):
        if not self._settled:
            self._settled = True
            self._box._finished(self)


class BoxRunner:
    """Routes ``submit_state_once`` over several replicas (``scheduler.BatchHandle``, one per GPU)."""

    def __init__(self, handles: Sequence[BatchHandle], owner_entries: int = 1 << 16):
        if not handles:
            raise ValueError("a box needs at least one replica")
        self.handles = list(handles)
        self.world = len(self.handles)
        self._lock = threading.Lock()
        self._owner: "OrderedDict[bytes, int]" = OrderedDict()  # state key -> the replica that holds (or held) its capture
        self._owner_entries = owner_entries
        self._open: list[list[BoxTicket]] = [[] for _ in self.handles]
        self.requests = [0] * self.world
        self.affinity_hits = [0] * self.world
        self.steals = [0] * self.world   # cold states taken by a replica that is not their static home

    def in_flight(self) -> list[int]:
        with self._lock:
            self._prune()
            return [len(o) for o in self._open]

    def _prune(self):
        for o in self._open:
            o[:] = [t for t in o if not t._settled and not t.done()]

    def _finished(self, ticket: BoxTicket):
        with self._lock:
            o = self._open[ticket.replica]
            if ticket in o:
                o.remove(ticket)

    def route(self, key: bytes) -> tuple[int, bool, bool]:
        """(replica, affinity hit, stolen) for a state key; call with the lock held."""
        r = self._owner.get(key)
        if r is not None:
            return r, True, False
        home = state_affinity_rank(key, self.world)
        load = [len(o) for o in self._open]
        least = min(load)
        r = home if load[home] == least else load.index(least)
        return r, False, r != home

    def submit_state_once(self, state: Sequence[int], questions: Sequence[Sequence[int]], digest: bytes | None = None) -> BoxTicket:
        """Same arguments as ``BatchHandle.submit_state_once``; returns at once. Raises what the chosen replica raises
        (EngineError(E_OVERLOADED) when its queue is full)."""
        key = state_key(state, digest)
        with self._lock:
            self._prune()
            r, hit, stolen = self.route(key)
            ticket = BoxTicket(self, self.handles[r].submit_state_once(state, questions, digest), r, stolen)
            self._owner[key] = r  # only once the replica has taken the request
            self._owner.move_to_end(key)
            if len(self._owner) > self._owner_entries:
                self._owner.popitem(last=False)
            self._open[r].append(ticket)
            self.requests[r] += 1
            self.affinity_hits[r] += int(hit)
            self.steals[r] += int(stolen)
        return ticket

    def stats(self) -> dict:
        with self._lock:
            out = {"replicas": self.world, "requests": list(self.requests), "affinity_hits": list(self.affinity_hits), "steals": list(self.steals)}
        out["schedulers"] = [h.stats() for h in self.handles]
        return out

    def close(self):
        for h in self.handles:
            h.close()
