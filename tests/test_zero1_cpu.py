"""CPU: host-side ZeRO-1 logic (partitioning, slice bounds) and its agreement across ranks,
run as two gloo processes; no GPU and no NCCL involved."""
import os

import numpy as np
import pytest

from ancora_cutile_b200 import shapes as S
from ancora_cutile_b200.hybrid import default_is_muon, muon_names_for
from ancora_cutile_b200.zero1 import greedy_partition, ns_cost, slice_bounds


def _muon_costs():
    shp = S.qwen3_0_6b_shapes()
    mu = muon_names_for(shp)
    return shp, mu, [ns_cost(*shp[n]) for n in mu]


def test_ns_cost_counts_flops_of_one_iteration():
    assert ns_cost(1024, 3072) == ns_cost(3072, 1024) == 4 * 1024 ** 2 * 3072 + 2 * 1024 ** 3


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_greedy_partition_balanced_and_deterministic(world):
    _, mu, costs = _muon_costs()
    owner, load = greedy_partition(costs, world)
    assert owner == greedy_partition(costs, world)[0]
    assert sorted(set(owner)) == list(range(world))
    assert max(load) <= 1.02 * sum(load) / world
    assert sum(load) == sum(costs)


def test_slice_bounds():
    per, padded = slice_bounds(155_648_000, 8)
    assert per % 64 == 0 and padded == 8 * per and padded >= 155_648_000 and padded - 155_648_000 < 8 * 64
    assert slice_bounds(10, 4) == (64, 256)
    assert slice_bounds(64, 1) == (64, 64)


def _worker(rank, world, port, q):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    shp, mu, costs = _muon_costs()
    owner, _ = greedy_partition(costs, world)
    a_total = sum(int(np.prod(s)) for n, s in shp.items() if n not in set(mu))
    per, padded = slice_bounds(a_total, world)
    mine = dict(rank=rank, owner=owner, slice=(rank * per, (rank + 1) * per), padded=padded,
                my_matrices=[n for n, o in zip(mu, owner) if o == rank])
    box = [None] * world
    dist.all_gather_object(box, mine)
    if rank == 0:
        q.put(box)
    dist.barrier()
    dist.destroy_process_group()


def test_two_ranks_agree_and_cover_everything():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + (os.getpid() % 2000)
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    box = q.get(timeout=120)
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    assert box[0]["owner"] == box[1]["owner"]
    assert box[0]["slice"][1] == box[1]["slice"][0] and box[1]["slice"][1] == box[0]["padded"]
    _, mu, _ = _muon_costs()
    assert sorted(box[0]["my_matrices"] + box[1]["my_matrices"]) == sorted(mu)
    assert not set(box[0]["my_matrices"]) & set(box[1]["my_matrices"])


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_partition_by_group_counts_and_balance(world):
    from ancora_cutile_b200.zero1 import partition_by_group
    for shp in (S.qwen3_0_6b_shapes(), S.moe_family_shapes()):
        mu = muon_names_for(shp)
        shapes = [shp[n] for n in mu]
        owner, load = partition_by_group(shapes, world)
        assert owner == partition_by_group(shapes, world)[0]
        assert sum(load) == sum(ns_cost(*s) for s in shapes)
        assert max(load) <= 1.03 * sum(load) / world
        groups = {}
        for s, o in zip(shapes, owner):
            groups.setdefault((min(s), max(s)), []).append(o)
        for key, owners in groups.items():
            counts = [owners.count(r) for r in range(world)]
            assert max(counts) - min(counts) <= 1, (key, counts)        # floor or ceil per rank
            assert owners == sorted(owners)                              # contiguous runs in registration order
