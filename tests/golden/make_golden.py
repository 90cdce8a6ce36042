"""Generates the committed oracle fixtures.

tests/golden/tiny_oracle.npz: logits of the CPU oracle on BASELINE config 1 (tiny hybrid,
seed 0, one 128-token state, questions of 16/20/24/32 tokens; ids from PCG64(0)), in f32 and bf16 modes.

tests/golden/d3_slice_oracle.npz (``--d3``, a few minutes of CPU): a 4-layer [GDN,GDN,GDN,full] slice at
d3-turbo dimensions, one 96-token state and questions of 20/33/48/17 tokens (PCG64(11), vocab 8192):
bf16 logits with the default GEMM summation order (v0), bf16 logits with double-precision in-order
accumulation (v1) and f32 logits. v0 vs v1 measures how far bf16 logits move when only the summation
order changes, i.e. the noise floor any independent bf16 implementation sits on.

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


if __name__ == "__main__":
    if "--d3" in sys.argv:
        d3_slice()
    else:
        main()
