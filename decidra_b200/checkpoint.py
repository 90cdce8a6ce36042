"""Checkpoint access: the host-side mirror of juanqui/decidra's ``Store`` (native/src/tensor.rs),
``Config::from_dir`` (native/src/config.rs) and the ``Engine::new`` + ``preload_all`` start-up
sequence (native/src/engine.rs:791-870, 1265-1300), over the C ABI of ``libdecidra_b200.so``.

The store memory-maps the safetensors shards and copies nothing; ``Engine.load_checkpoint`` streams
the tensors to the device and converts the stored formats there.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import numpy as np

from . import _lib
from .config import ModelConfig, Options
from .engine import Engine, EngineError

DT_F32, DT_F16, DT_BF16, DT_I32, DT_I64, DT_U8, DT_F8E4M3 = range(7)
# numpy views of the stored bytes; BF16 has no numpy type and is exposed as uint16 bit patterns
_NP = {DT_F32: np.float32, DT_F16: np.float16, DT_BF16: np.uint16, DT_I32: np.int32, DT_I64: np.int64, DT_U8: np.uint8,
       DT_F8E4M3: np.uint8}


def _last_error() -> str:
    return (_lib.load().dcd_last_error(None) or b"").decode()


class Store:
    """``Store::open`` / ``Store::open_file``: a model directory or a single ``.safetensors`` file."""

    def __init__(self, path):
        self._h = None
        out = C.c_void_p()
        rc = _lib.load().dcd_checkpoint_open(str(path).encode(), C.byref(out))
        if rc:
            raise EngineError(rc, _last_error())
        self._h = out

    def close(self):
        if self._h:
            _lib.load().dcd_checkpoint_close(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def __len__(self) -> int:
        return int(_lib.load().dcd_checkpoint_count(self._h))

    def names(self):
        lib = _lib.load()
        return [lib.dcd_checkpoint_name(self._h, i).decode() for i in range(len(self))]

    def contains(self, name: str) -> bool:
        info = _lib.TensorInfo()
        return _lib.load().dcd_checkpoint_tensor(self._h, name.encode(), C.byref(info)) == 0

    def info(self, name: str):
        """(dtype code, shape tuple, byte count) or raise if absent."""
        info = _lib.TensorInfo()
        rc = _lib.load().dcd_checkpoint_tensor(self._h, name.encode(), C.byref(info))
        if rc:
            raise EngineError(rc, _last_error())
        return int(info.dtype), tuple(int(info.shape[i]) for i in range(info.rank)), int(info.bytes)

    def array(self, name: str) -> np.ndarray:
        """A copy of the stored tensor (BF16 as uint16 bit patterns, F8 as raw bytes)."""
        info = _lib.TensorInfo()
        rc = _lib.load().dcd_checkpoint_tensor(self._h, name.encode(), C.byref(info))
        if rc:
            raise EngineError(rc, _last_error())
        shape = tuple(int(info.shape[i]) for i in range(info.rank))
        if info.bytes == 0:
            return np.empty(shape, dtype=_NP[info.dtype])
        buf = C.string_at(info.data, info.bytes)
        return np.frombuffer(buf, dtype=_NP[info.dtype]).reshape(shape).copy()


def config_from_dir(model_dir) -> ModelConfig:
    """``Config::from_dir``; ``readout_rows`` is left 0 (set it from the readout head)."""
    cfg = ModelConfig()
    rc = _lib.load().dcd_config_from_dir(str(model_dir).encode(), C.byref(cfg))
    if rc:
        raise EngineError(rc, _last_error())
    return cfg


def load_checkpoint(engine: Engine, store: Store, readout_path=None) -> None:
    """``preload_all``: every weight of ``engine`` from ``store`` (+ the separate readout head)."""
    rp = None if readout_path is None else str(readout_path).encode()
    engine._check(_lib.load().dcd_engine_load_checkpoint(engine._h, store._h, rp))


def load_tensor_typed(engine: Engine, layer: int, kind: int, values: np.ndarray, dtype: int) -> None:
    """Upload one tensor in its stored type (``values``: f32, f16, or uint16 bf16 bit patterns)."""
    v = np.ascontiguousarray(values).ravel()
    engine._check(_lib.load().dcd_engine_load_tensor_typed(engine._h, layer, kind, v.ctypes.data_as(C.c_void_p), dtype, v.size))


def engine_from_dir(model_dir, options: Options | None = None, device: int = 0) -> Engine:
    """``Engine::new(model_dir)`` followed by ``preload_all``: config.json (+ decision_config.json),
    the safetensors shards and ``readout.safetensors`` of one model directory."""
    model_dir = Path(model_dir)
    cfg = config_from_dir(model_dir)
    readout = model_dir / "readout.safetensors"
    head = Store(readout)
    try:
        _, shape, _ = head.info("weight")
    finally:
        head.close()
    if len(shape) != 2:
        raise EngineError(_lib.E_INVALID, f"readout.weight must be 2-D, got {list(shape)}")
    cfg.readout_rows = shape[0]
    engine = Engine(cfg, options, device)
    store = Store(model_dir)
    try:
        load_checkpoint(engine, store, readout)
    finally:
        store.close()
    return engine
