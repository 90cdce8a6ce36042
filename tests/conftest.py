import os
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def oracle():
    """The CPU oracle (test infrastructure), built on demand with g++."""
    from oracle import cpu_oracle
    cpu_oracle.build()
    cpu_oracle.lib()
    return cpu_oracle


@pytest.fixture(scope="session")
def dcd():
    """The product package; the CUDA library must already be built in-tree."""
    import decidra_b200
    from decidra_b200 import _lib
    if not _lib.LIB_PATH.exists():
        from decidra_b200 import build
        build.build()
    _lib.load()
    return decidra_b200


def orc_cfg(oracle, cfg):
    """Oracle config with the same fields as a product ModelConfig."""
    return oracle.make_config(
        num_layers=cfg.num_layers, hidden=cfg.hidden, heads=cfg.heads, kv_heads=cfg.kv_heads, head_dim=cfg.head_dim,
        rotary_dim=cfg.rotary_dim, rope_theta=cfg.rope_theta, gdn_k_heads=cfg.gdn_k_heads, gdn_v_heads=cfg.gdn_v_heads,
        gdn_dk=cfg.gdn_dk, gdn_dv=cfg.gdn_dv, conv_kernel=cfg.conv_kernel, intermediate=cfg.intermediate, vocab=cfg.vocab,
        readout_rows=cfg.readout_rows, rms_eps=cfg.rms_eps, dtype=cfg.dtype, layer_is_full=cfg.layer_types())


def tiny_inputs(seed=0, vocab=4096, state_len=128, qlens=(16, 20, 24, 32)):
    rng = np.random.Generator(np.random.PCG64(seed))
    state = rng.integers(0, vocab, state_len, dtype=np.uint32)
    questions = [rng.integers(0, vocab, n, dtype=np.uint32) for n in qlens]
    return state, questions
