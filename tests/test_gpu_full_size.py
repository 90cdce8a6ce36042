"""The full 64-layer d3-shaped model at the sizes of the ragged-stress benchmark workload ( long states, many questions of
16-512 tokens), where the CPU oracle is out of reach: size-independent properties instead. A permuted batch must
give the same rows (the chunk planner sorts and cuts the batch, rows go back to input order), a state that went
through pinned host memory must answer identically, and one pass over several states must equal a pass per state.
All comparisons are bit-exact."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def full(dcd):
    import torch
    if torch.cuda.get_device_properties(0).total_memory < 120 * 2**30:
        pytest.skip("needs the 54 GB of bf16 weights plus workspace")
    o = dcd.Options()
    o.max_pass_tokens = 16384
    e = dcd.Engine(dcd.d3_config(), o)
    e.init_random(0)
    yield e
    e.close()


def test_ragged_stress_properties_at_full_size(dcd, full):
    e = full
    vocab = e.cfg.vocab
    rng = np.random.Generator(np.random.PCG64(7))
    # a long state with a moderate batch, and a short state with a batch that needs several passes
    for S, nq in ((10393, 48), (1133, 150)):
        state = rng.integers(0, vocab, S, dtype=np.uint32)
        qs = [rng.integers(0, vocab, int(n), dtype=np.uint32) for n in rng.integers(16, 513, nq)]
        c = e.capture_state(state)
        out = e.readout_state_once_batch(c, qs)
        assert out.shape == (nq, 255) and np.isfinite(out).all()
        assert np.abs(out).max() > 1e-3 and len(np.unique(out.argmax(1))) > 1          # not a constant answer
        perm = rng.permutation(nq)
        assert e.readout_state_once_batch(c, [qs[i] for i in perm]).tobytes() == out[perm].tobytes()
        host = c.offload()
        c2 = dcd.StateCache.restore(host, e)
        assert e.readout_state_once_batch(c2, qs[:8]).tobytes() == out[:8].tobytes()
        c.free(); c2.free(); host.free()


def test_multi_state_equals_per_state_at_full_size(dcd, full):
    e = full
    vocab = e.cfg.vocab
    rng = np.random.Generator(np.random.PCG64(11))
    states = [rng.integers(0, vocab, n, dtype=np.uint32) for n in (2048, 700, 4100)]
    caches = [e.capture_state(s) for s in states]
    state_of = rng.integers(0, 3, 40).astype(np.uint32)
    qs = [rng.integers(0, vocab, int(n), dtype=np.uint32) for n in rng.integers(16, 300, 40)]
    got = e.readout_multi_state_batch(caches, qs, state_of)
    for k, c in enumerate(caches):
        idx = [i for i in range(40) if state_of[i] == k]
        assert got[idx].tobytes() == e.readout_state_once_batch(c, [qs[i] for i in idx]).tobytes(), k
    for c in caches:
        c.free()
