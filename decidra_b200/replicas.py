"""Data-parallel replicas sharded by state (no tensor parallelism, no collective on the hot path).

Every question attends only to its own state's cache, so a state and all its questions go to one
replica; the reference's own cache key is exactly (state ids, image digest) (src/batch.rs:506-513 in
juanqui/decidra), and it already processes state groups independently (src/batch.rs:499-503). Each
replica is one process / one engine / one GPU holding a full copy of the weights.
"""
from __future__ import annotations

import hashlib

import numpy as np


def state_affinity_rank(state_key: bytes, world: int) -> int:
    """Static routing for cache affinity: the same state always lands on the same replica."""
    return int.from_bytes(hashlib.blake2b(state_key, digest_size=8).digest(), "little") % world


def shard_states(costs, world: int, rank: int) -> np.ndarray:
    """Indices of the states this rank owns. Greedy longest-processing-time assignment on the predicted
    cost (FLOPs of capture + questions), so ragged workloads balance by work, not by count."""
    costs = np.asarray(costs, dtype=np.float64)
    order = np.argsort(-costs, kind="stable")
    load = np.zeros(world)
    owner = np.empty(len(costs), dtype=np.int64)
    for i in order:
        r = int(np.argmin(load))
        owner[i] = r
        load[r] += costs[i]
    return np.nonzero(owner == rank)[0]


def synthetic_costs(n_states: int, seed: int = 7) -> np.ndarray:
    """Cost proxy of a ragged mix: state length log-uniform in [256,16384] times a question count."""
    rng = np.random.Generator(np.random.PCG64(seed))
    S = np.exp(rng.uniform(np.log(256), np.log(16384), n_states))
    B = rng.integers(1, 257, n_states)
    return S + B * 264.0
