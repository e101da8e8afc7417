"""Multi-rank host logic on CPU: partitioning and the optional gather of reconstructed shards,
exercised with world_size = 2 over gloo."""
from __future__ import annotations

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from ade_b200 import sharding


def test_llama_shapes_and_partition_balance():
    shapes = sharding.llama_module_shapes(5120, 13824, 40)
    assert len(shapes) == 280 and shapes[0] == ("model.layers.0.self_attn.q_proj", 5120, 5120)
    assert shapes[6] == ("model.layers.0.mlp.down_proj", 5120, 13824)
    costs = [a * b for _, a, b in shapes]
    for world in (1, 2, 4, 8):
        plan = sharding.partition_modules(costs, world)
        assert sorted(i for p in plan for i in p) == list(range(280))
        loads = [sum(costs[i] for i in p) for p in plan]
        assert max(loads) / (sum(loads) / world) < 1.02            # within 2 % of perfect balance
    assert sharding.partition_modules([5, 5, 5], 2) == [[0, 2], [1]]
    assert sharding.replica_plan(8, 8) == [[i] for i in range(8)]
    assert sharding.replica_plan(8, 2) == [[0, 2, 4, 6], [1, 3, 5, 7]]
    with pytest.raises(ValueError):
        sharding.partition_modules([1], 0)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        dims = [(4, 6), (8, 2), (2, 2), (6, 6), (2, 10)]
        shapes = dict(enumerate(dims))
        plan = sharding.partition_modules([a * b for a, b in dims], world)
        # stand-in for the reconstruction kernel: module i is filled with i + 1
        local = {i: torch.full(dims[i], float(i + 1), dtype=torch.bfloat16) for i in plan[rank]}
        full = sharding.gather_merged(local, shapes, plan)
        ok = sorted(full) == list(range(len(dims))) and all(
            tuple(full[i].shape) == dims[i] and bool((full[i] == i + 1).all()) for i in full)
        bad = False
        try:
            sharding.gather_merged({}, shapes, plan) if plan[rank] else None
        except ValueError:
            bad = True
        q.put((rank, ok, bad or not plan[rank]))
    finally:
        dist.destroy_process_group()


def test_gather_merged_two_ranks():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert all(ok and bad for _, ok, bad in res), res
