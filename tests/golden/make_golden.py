"""Generates the committed oracle fixtures.

tests/golden/tiny_oracle.npz: logits of the CPU oracle on the tiny CPU-runnable benchmark model (tiny hybrid,
seed 0, one 128-token state, questions of 16/20/24/32 tokens; ids from PCG64(0)), in f32 and bf16 modes.

tests/golden/d3_slice_oracle.npz (``--d3``, a few minutes of CPU): a 4-layer [GDN,GDN,GDN,full] slice at
d3-turbo dimensions, one 96-token state and questions of 20/33/48/17 tokens (PCG64(11), vocab 8192):
bf16 logits with the default GEMM summation order (v0), bf16 logits with double-precision in-order
accumulation (v1) and f32 logits. v0 vs v1 measures how far bf16 logits move when only the summation
order changes, i.e. the noise floor any independent bf16 implementation sits on.

tests/golden/d3_argmax_oracle.npz (``--d3-argmax``, ~20 minutes of CPU): the same 4-layer slice, one 64-token state and 256
questions of 8..24 tokens (PCG64(23), vocab 8192): bf16 and f32 logits [256, 255]. Enough rows to put a number on the
">= 99.5 % per-question argmax agreement" bar (4 questions cannot).

tests/golden/d3_64layer_oracle.npz (``--d3-64``, ~10 minutes of CPU): the full 64-layer d3-shaped model (vocab 248320), one
64-token state and 4 questions of 48 tokens (PCG64(29)); the oracle generates each layer's weights when the pass reaches
it. bf16 logits [4, 255], the residual stream after layers 8, 16, ..., 64 at each question's last row [8, 4, 5120], and
layer 63's cached K (first 8 state rows) / layer 62's recurrent state (first value head).

The fixtures pin the oracle against itself across rebuilds and machines (same compiler flags, no FMA
contraction). They are NOT reference goldens: the reference needs its checkpoint and a GPU to produce
model-level outputs, and neither is available. Run:  python tests/golden/make_golden.py [--d3]
"""
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))

from conftest import orc_cfg, tiny_inputs  # noqa: E402
from decidra_b200.config import tiny_config  # noqa: E402
from oracle import cpu_oracle as O  # noqa: E402


def main():
    state, questions = tiny_inputs()
    out = {"state": state, "qlens": np.array([len(q) for q in questions]), "questions": np.concatenate(questions)}
    for name, dt in (("f32", 0), ("bf16", 1)):
        o = O.Oracle(orc_cfg(O, tiny_config(dt)), 0)
        st = o.capture_state(state)
        out[f"logits_{name}"] = o.readout_state_once_batch(st, questions)
        out[f"gdn_state0_{name}"] = st.tensor(0, 2)
        out[f"k3_{name}"] = st.tensor(3, 0)
    np.savez_compressed(Path(__file__).with_name("tiny_oracle.npz"), **out)
    print({k: v.shape for k, v in out.items()})


def d3_slice():
    from decidra_b200.config import d3_config
    state, questions = tiny_inputs(seed=11, vocab=8192, state_len=96, qlens=(20, 33, 48, 17))
    out = {}
    for name, dt, variant in (("bf16_v0", 1, 0), ("bf16_v1", 1, 1), ("f32", 0, 1)):
        O.lib().orc_set_gemm_variant(variant)
        o = O.Oracle(orc_cfg(O, d3_config(num_layers=4, dtype=dt, vocab=8192)), 0)
        out[f"logits_{name}"] = o.readout_state_once_batch(o.capture_state(state), questions)
        del o
    O.lib().orc_set_gemm_variant(0)
    np.savez_compressed(Path(__file__).with_name("d3_slice_oracle.npz"), **out)
    print({k: float(np.abs(v - out["logits_f32"]).max()) for k, v in out.items()})


def argmax_inputs():
    rng = np.random.Generator(np.random.PCG64(23))
    state = rng.integers(0, 8192, 64, dtype=np.uint32)
    lens = rng.integers(8, 25, 256)
    return state, [rng.integers(0, 8192, int(n), dtype=np.uint32) for n in lens]


def d3_argmax():
    from decidra_b200.config import d3_config
    state, questions = argmax_inputs()
    out = {}
    for name, dt in (("bf16", 1), ("f32", 0)):
        o = O.Oracle(orc_cfg(O, d3_config(num_layers=4, dtype=dt, vocab=8192)), 0)
        out[f"logits_{name}"] = o.readout_state_once_batch(o.capture_state(state), questions)
        del o
    np.savez_compressed(Path(__file__).with_name("d3_argmax_oracle.npz"), **out)
    d = np.abs(out["logits_bf16"] - out["logits_f32"])
    print("bf16 vs f32 max-abs", float(d.max()), "argmax agree", float((out["logits_bf16"].argmax(1) == out["logits_f32"].argmax(1)).mean()))


def deep_inputs():
    rng = np.random.Generator(np.random.PCG64(29))
    state = rng.integers(0, 248320, 64, dtype=np.uint32)
    return state, [rng.integers(0, 248320, 48, dtype=np.uint32) for _ in range(4)]


def d3_64():
    from decidra_b200.config import d3_config
    state, questions = deep_inputs()
    cfg = d3_config(num_layers=64, dtype=1)
    o = O.Oracle(orc_cfg(O, cfg), 0, lazy=True)
    st = o.capture_state(state)
    o.tap_enable(True)
    logits = o.readout_state_once_batch(st, questions)
    H = cfg.hidden
    last = np.cumsum([len(q) for q in questions]) - 1
    rows = np.stack([o.tap(f"layer_out_{li}").reshape(-1, H)[last] for li in range(7, 64, 8)])
    out = {"logits_bf16": logits, "layer_out_last_rows": rows, "k63_head": st.tensor(63, 0)[:8 * 4 * 256],
           "gdn_state62_head0": st.tensor(62, 2)[:128 * 128]}
    np.savez_compressed(Path(__file__).with_name("d3_64layer_oracle.npz"), **out)
    print({k: v.shape for k, v in out.items()}, float(np.abs(logits).max()))


if __name__ == "__main__":
    if "--d3-argmax" in sys.argv:
        d3_argmax()
    elif "--d3-64" in sys.argv:
        d3_64()
    elif "--d3" in sys.argv:
        d3_slice()
    else:
        main()
