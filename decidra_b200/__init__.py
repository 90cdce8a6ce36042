"""decidra_b200: B200-native (sm_100a) state-once question path behind the reference's Engine API.

The compute lives in ``libdecidra_b200.so`` (hand-written CUDA, see ``csrc/``); this package is the
thin host mirror of the reference interface. There is no CPU fallback.
"""
from .config import ModelConfig, Options, d3_config, make_config, tiny_config
from .engine import Engine, EngineError, HostStateCache, StateCache
from . import checkpoint  # noqa: E402  (Store, config_from_dir, engine_from_dir)
from . import prompt, scheduler  # noqa: E402

__all__ = ["ModelConfig", "Options", "d3_config", "make_config", "tiny_config", "Engine", "EngineError", "HostStateCache", "StateCache", "checkpoint", "prompt", "scheduler"]
