"""The multi-GPU path is replicas sharded by state with no data-path collective. These CPU tests run
the sharding logic as two gloo ranks: every state lands on exactly one rank and the whole-job count is
the sum of the ranks' counts."""
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, n_states, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from decidra_b200 import replicas
    costs = replicas.synthetic_costs(n_states, seed=7)
    mine = replicas.shard_states(costs, world, rank)
    owned = torch.zeros(n_states, dtype=torch.int64)
    owned[mine] = 1
    dist.all_reduce(owned)
    count = torch.tensor([len(mine)], dtype=torch.int64)
    dist.all_reduce(count)
    t = torch.tensor([float(costs[mine].sum())], dtype=torch.float64)
    tmax = t.clone()
    dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
    if rank == 0:
        np.savez(Path(out_dir) / "r.npz", owned=owned.numpy(), count=count.numpy(), tmax=tmax.numpy(), total=float(costs.sum()))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("n_states", [8, 37])
def test_states_shard_disjointly_over_two_ranks(tmp_path, n_states):
    port = _free_port()
    mp.spawn(_worker, args=(2, port, n_states, str(tmp_path)), nprocs=2, join=True)
    r = np.load(tmp_path / "r.npz")
    assert (r["owned"] == 1).all()            # each state on exactly one rank
    assert int(r["count"][0]) == n_states
    assert r["tmax"][0] <= 0.5 * r["total"] * 1.25 + 1e-9   # cost-balanced within 25 %


def test_shard_states_properties():
    from decidra_b200 import replicas
    costs = replicas.synthetic_costs(100, seed=1)
    seen = np.zeros(100, int)
    for world in (1, 2, 4, 8):
        seen[:] = 0
        for rank in range(world):
            seen[replicas.shard_states(costs, world, rank)] += 1
        assert (seen == 1).all()
    assert list(replicas.shard_states(np.ones(8), 8, 3)) == [3]
    assert replicas.state_affinity_rank(b"abc", 8) == replicas.state_affinity_rank(b"abc", 8)
