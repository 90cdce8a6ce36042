"""Host-side mirror of the reference's ``Engine`` / ``StateCache`` interface for the state-once path.

Same names, argument meaning and error behaviour as juanqui/decidra's ``decidra_native`` crate
(native/src/engine.rs): ``Engine.capture_state``, ``Engine.readout_state_once_batch``,
``Engine.decision_logits_split``, ``StateCache.offload`` / ``restore``. Everything below these calls
runs in ``libdecidra_b200.so`` on the GPU; this module only marshals host buffers through the C ABI.
"""
from __future__ import annotations

import ctypes as C
from typing import Sequence

import numpy as np

from . import _lib
from .config import ModelConfig, Options


class EngineError(RuntimeError):
    """Raised for any non-zero status of the C ABI; ``code`` is the DCD_E_* value. Out-of-memory
    messages contain "out of memory", the substring the reference scheduler retries on
    (src/batch.rs:767,863)."""

    def __init__(self, code: int, message: str):
        super().__init__(message)
        self.code = code


def _u32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.uint32)


class HostStateCache:
    """``HostStateCache`` (native/src/engine.rs:545-551): a pinned host copy of a StateCache."""

    def __init__(self, engine: "Engine", handle):
        self._engine, self._h = engine, handle

    def free(self):
        if self._h:
            _lib.load().dcd_host_state_free(self._h)
            self._h = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class StateCache:
    """``StateCache`` (native/src/engine.rs:533-543): per-layer post-RoPE K and raw V of the state on
    full-attention layers, final f32 recurrent state and 3-row conv tail on GDN layers."""

    def __init__(self, engine: "Engine", handle):
        self._engine, self._h = engine, handle

    @property
    def state_len(self) -> int:
        return int(_lib.load().dcd_state_tokens(self._h))

    def state_tokens(self) -> int:
        return self.state_len

    @property
    def pos_end(self) -> int:
        return int(_lib.load().dcd_state_pos_end(self._h))

    @property
    def nbytes(self) -> int:
        return int(_lib.load().dcd_state_bytes(self._h))

    def offload(self) -> HostStateCache:
        out = C.c_void_p()
        self._engine._check(_lib.load().dcd_state_offload(self._engine._h, self._h, C.byref(out)))
        return HostStateCache(self._engine, out)

    @staticmethod
    def restore(host: HostStateCache, engine: "Engine") -> "StateCache":
        out = C.c_void_p()
        engine._check(_lib.load().dcd_state_restore(engine._h, host._h, C.byref(out)))
        return StateCache(engine, out)

    def zero_gdn_state(self, layer: int) -> None:
        self._engine._check(_lib.load().dcd_state_zero_gdn_state(self._engine._h, self._h, layer))

    def zero_gdn_hist(self, layer: int) -> None:
        self._engine._check(_lib.load().dcd_state_zero_gdn_hist(self._engine._h, self._h, layer))

    def tensor(self, layer: int, what: int):
        """what: 0 K, 1 V, 2 recurrent state, 3 conv tail; returns f32 or None if the layer has none."""
        n = C.c_size_t()
        rc = _lib.load().dcd_state_read_tensor(self._engine._h, self._h, layer, what, None, C.byref(n))
        if rc:
            return None
        out = np.empty(n.value, dtype=np.float32)
        self._engine._check(_lib.load().dcd_state_read_tensor(self._engine._h, self._h, layer, what, out.ctypes.data_as(_lib.FP), C.byref(n)))
        return out

    def free(self):
        if self._h and self._engine._h:
            _lib.load().dcd_state_free(self._engine._h, self._h)
        self._h = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class Engine:
    """One engine = one GPU, one stream, one caller thread (native/src/engine.rs:374-377)."""

    def __init__(self, cfg: ModelConfig, options: Options | None = None, device: int = 0):
        self._h = None
        lib = _lib.load()
        self.cfg = cfg
        self.options = options or Options()
        out = C.c_void_p()
        rc = lib.dcd_engine_create(C.byref(cfg), C.byref(self.options), device, C.byref(out))
        if rc:
            raise EngineError(rc, (lib.dcd_last_error(None) or b"").decode())
        self._h = out

    # -- lifecycle ----------------------------------------------------------------------------
    def close(self):
        if self._h:
            _lib.load().dcd_engine_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _check(self, rc: int):
        if rc:
            raise EngineError(rc, (_lib.load().dcd_last_error(self._h) or b"").decode())

    def info(self) -> _lib.Info:
        out = _lib.Info()
        self._check(_lib.load().dcd_engine_info(self._h, C.byref(out)))
        return out

    def init_random(self, seed: int = 0) -> None:
        """Stands where ``preload_all`` loads the checkpoint: seeded random-init weights."""
        self._check(_lib.load().dcd_engine_init_random(self._h, seed))

    def load_tensor(self, layer: int, kind: int, values) -> None:
        v = np.ascontiguousarray(values, dtype=np.float32).ravel()
        self._check(_lib.load().dcd_engine_load_tensor(self._h, layer, kind, v.ctypes.data_as(_lib.FP), v.size))

    def read_tensor(self, layer: int, kind: int, count: int) -> np.ndarray:
        out = np.empty(count, dtype=np.float32)
        self._check(_lib.load().dcd_engine_read_tensor(self._h, layer, kind, out.ctypes.data_as(_lib.FP), count))
        return out

    def rebind_blas(self) -> None:
        self._check(_lib.load().dcd_rebind_blas(self._h))

    # -- hot path -----------------------------------------------------------------------------
    def capture_state(self, tokens: Sequence[int]) -> StateCache:
        """``Engine::capture_state`` (native/src/engine.rs:4607-4610): once per state."""
        ids = _u32(tokens)
        out = C.c_void_p()
        self._check(_lib.load().dcd_capture_state(self._h, ids.ctypes.data_as(_lib.U32P), ids.size, None, C.byref(out)))
        return StateCache(self, out)

    def readout_state_once_batch(self, cache: StateCache, questions: Sequence[Sequence[int]]) -> np.ndarray:
        """``Engine::readout_state_once_batch`` (native/src/engine.rs:4847-4861): [B, readout_rows] f32
        logits in input order."""
        B = len(questions)
        arrs = [_u32(q) for q in questions]
        ptrs = (_lib.U32P * max(B, 1))(*[a.ctypes.data_as(_lib.U32P) for a in arrs])
        lens = (C.c_size_t * max(B, 1))(*[a.size for a in arrs])
        out = np.empty((B, self.cfg.readout_rows), dtype=np.float32)
        self._check(_lib.load().dcd_readout_state_once_batch(self._h, cache._h, ptrs, lens, B, out.ctypes.data_as(_lib.FP)))
        return out

    def capture_and_readout(self, state: Sequence[int], questions: Sequence[Sequence[int]]):
        """A cold request in one pass (``dcd_capture_and_readout``): returns ``(StateCache, logits [B, readout_rows])``, bit-identical
        to ``capture_state`` followed by ``readout_state_once_batch``; the library falls back to that order when one pass cannot
        hold the request."""
        ids = _u32(state)
        B = len(questions)
        arrs = [_u32(q) for q in questions]
        ptrs = (_lib.U32P * max(B, 1))(*[a.ctypes.data_as(_lib.U32P) for a in arrs])
        lens = (C.c_size_t * max(B, 1))(*[a.size for a in arrs])
        out = np.empty((B, self.cfg.readout_rows), dtype=np.float32)
        st = C.c_void_p()
        self._check(_lib.load().dcd_capture_and_readout(self._h, ids.ctypes.data_as(_lib.U32P), ids.size, ptrs, lens, B, C.byref(st),
                                                        out.ctypes.data_as(_lib.FP)))
        return StateCache(self, st), out

    def readout_multi_state_batch(self, caches: Sequence[StateCache], questions: Sequence[Sequence[int]], state_of: Sequence[int]) -> np.ndarray:
        """One pass over questions of several states: ``state_of[i]`` indexes ``caches``. Rows equal those of
        ``readout_state_once_batch`` per state, bit for bit; [B, readout_rows] f32 in input order."""
        B = len(questions)
        arrs = [_u32(q) for q in questions]
        ptrs = (_lib.U32P * max(B, 1))(*[a.ctypes.data_as(_lib.U32P) for a in arrs])
        lens = (C.c_size_t * max(B, 1))(*[a.size for a in arrs])
        handles = (C.c_void_p * max(len(caches), 1))(*[c._h.value for c in caches])
        sof = _u32(state_of)
        out = np.empty((B, self.cfg.readout_rows), dtype=np.float32)
        self._check(_lib.load().dcd_readout_multi_state_batch(self._h, handles, len(caches), ptrs, lens, sof.ctypes.data_as(_lib.U32P), B,
                                                              out.ctypes.data_as(_lib.FP)))
        return out

    def decision_logits_split(self, tokens: Sequence[int], split: int) -> np.ndarray:
        """``Engine::decision_logits_split`` (native/src/engine.rs:4585-4601): per-row reference."""
        ids = _u32(tokens)
        out = np.empty(self.cfg.readout_rows, dtype=np.float32)
        self._check(_lib.load().dcd_decision_logits_split(self._h, ids.ctypes.data_as(_lib.U32P), ids.size, split, out.ctypes.data_as(_lib.FP)))
        return out

    # device-resident forms (benchmarks): raw device pointers as ints
    def capture_state_device(self, d_ids: int, n: int) -> StateCache:
        out = C.c_void_p()
        self._check(_lib.load().dcd_capture_state_device(self._h, d_ids, n, C.byref(out)))
        return StateCache(self, out)

    def capture_and_readout_device(self, d_ids: int, d_lens: int, n_state: int, B: int, total: int, max_len: int, d_out: int) -> StateCache:
        out = C.c_void_p()
        self._check(_lib.load().dcd_capture_and_readout_device(self._h, d_ids, d_lens, n_state, B, total, max_len, C.byref(out), d_out))
        return StateCache(self, out)

    def readout_state_once_device(self, cache: StateCache, d_ids: int, d_lens: int, B: int, total: int, max_len: int, d_out: int) -> None:
        self._check(_lib.load().dcd_readout_state_once_device(self._h, cache._h, d_ids, d_lens, B, total, max_len, d_out))

    # -- pools, memory, timers ------------------------------------------------------------------
    def trim_pools(self) -> None:
        self._check(_lib.load().dcd_trim_pools(self._h))

    def mem_info(self):
        f, t = C.c_size_t(), C.c_size_t()
        self._check(_lib.load().dcd_mem_info(self._h, C.byref(f), C.byref(t)))
        return f.value, t.value

    def sync(self) -> None:
        self._check(_lib.load().dcd_engine_sync(self._h))

    def timer_begin(self) -> None:
        self._check(_lib.load().dcd_timer_begin(self._h))

    def timer_end(self) -> None:
        self._check(_lib.load().dcd_timer_end(self._h))

    def timer_seconds(self) -> float:
        return float(_lib.load().dcd_timer_seconds(self._h))

    def vision_encode(self, pixels=None):
        self._check(_lib.load().dcd_vision_encode(self._h, None, 0))

    def profile_enable(self, on: bool = True) -> None:
        self._check(_lib.load().dcd_profile_enable(self._h, int(on)))

    def profile_read(self) -> dict:
        arr = (_lib.ProfEntry * len(_lib.PROF_NAMES))()
        self._check(_lib.load().dcd_profile_read(self._h, arr))
        return {n: {"ms": arr[i].ms, "work": arr[i].work, "launches": arr[i].launches} for i, n in enumerate(_lib.PROF_NAMES)}

    def launch_count(self) -> int:
        return int(_lib.load().dcd_launch_count(self._h))

    def bounded_wait_probe(self, polls: int = 1024) -> None:
        """Make a bounded device-side wait run out on purpose (nothing arrives at its barrier): raises EngineError(E_TIMEOUT)."""
        self._check(_lib.load().dcd_debug_bounded_wait_probe(self._h, polls))

    def debug_layer_outputs(self, sink: np.ndarray | None) -> None:
        if sink is None:
            self._check(_lib.load().dcd_debug_layer_outputs(self._h, None, 0))
        else:
            assert sink.dtype == np.float32 and sink.flags.c_contiguous
            self._check(_lib.load().dcd_debug_layer_outputs(self._h, sink.ctypes.data_as(_lib.FP), sink.size))

    def pack(self, lens, pos_start: int):
        """Run the GPU packing kernel alone and return (cu_seqlens, positions, tok_q, last_row)."""
        lens = np.ascontiguousarray(lens, dtype=np.int32)
        B = lens.size
        total = int(np.clip(lens, 0, None).sum())
        cu = np.zeros(B + 1, np.int32)
        pos = np.zeros(max(total, 1), np.int32)
        tq = np.zeros(max(total, 1), np.int32)
        last = np.zeros(max(B, 1), np.int32)
        self._check(_lib.load().dcd_pack(self._h, lens.ctypes.data_as(_lib.I32P), B, pos_start, cu.ctypes.data_as(_lib.I32P),
                                         pos.ctypes.data_as(_lib.I32P), tq.ctypes.data_as(_lib.I32P), last.ctypes.data_as(_lib.I32P)))
        return cu, pos[:total], tq[:total], last[:B]
