"""Multi-GPU partitioning of the delta-application path.

Two workloads shard naturally, both without a collective on the data path:

* multi-delta serving -- one full replica of the base model plus one delta per GPU; the ranks never
  talk (``replica_plan``);
* whole-delta reconstruction -- the linear modules of one delta are independent units, split across
  ranks by longest-processing-time-first on the cost d_o * d_i (bytes dominate the kernel), see
  ``partition_modules``.  Each rank holds W_b and the packed delta only for its own modules.

``gather_merged`` is the one optional exchange: it assembles the reconstructed bf16 shards on every
rank with ``all_gather`` calls over the process group (NCCL over NVLink on GPUs, gloo in the CPU
tests).  It moves already-written tensors; nothing is fused with it.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from .serving import LINEAR_MODULE_NAMES


def llama_module_shapes(hidden: int, intermediate: int, layers: int, kv_hidden: int | None = None):
    """[(prefix, d_o, d_i)] of every delta-carrying linear module of a LLaMA-architecture model, in
    layer / name order (the order src/main.py:202-216 compresses them in)."""
    kv = hidden if kv_hidden is None else kv_hidden
    dims = {
        "self_attn.q_proj": (hidden, hidden), "self_attn.k_proj": (kv, hidden), "self_attn.v_proj": (kv, hidden),
        "self_attn.o_proj": (hidden, hidden), "mlp.gate_proj": (intermediate, hidden),
        "mlp.up_proj": (intermediate, hidden), "mlp.down_proj": (hidden, intermediate),
    }
    return [(f"model.layers.{li}.{n}", *dims[n]) for li in range(layers) for n in LINEAR_MODULE_NAMES]


def partition_modules(costs, world: int):
    """Longest-processing-time-first bin packing.  costs: list of numbers; returns a list of `world`
    lists of indices (each sorted), deterministic for equal inputs on every rank."""
    if world < 1:
        raise ValueError("world must be >= 1")
    order = sorted(range(len(costs)), key=lambda i: (-costs[i], i))
    load = [0.0] * world
    bins = [[] for _ in range(world)]
    for i in order:
        b = min(range(world), key=lambda j: (load[j], j))
        bins[b].append(i)
        load[b] += costs[i]
    return [sorted(b) for b in bins]


def replica_plan(n_deltas: int, world: int):
    """Delta ids served by each rank: round robin, one delta per GPU when n_deltas == world."""
    return [[d for d in range(n_deltas) if d % world == r] for r in range(world)]


def gather_merged(local: dict, shapes: dict, plan, group=None, device=None, dtype=torch.bfloat16):
    """Assemble reconstructed weights from all ranks.

    local:  {module index: merged tensor} of this rank (the modules plan[rank] lists).
    shapes: {module index: (d_o, d_i)} for every module.
    plan:   output of ``partition_modules``.
    device: where the exchange buffers live; default: the device of the local tensors, else the current
            CUDA device when the process group runs over NCCL, else the CPU.  A rank whose plan is empty has no
            local tensor to take it from, and NCCL needs its (empty-handed) contribution on a GPU as well.
    dtype:  element type of the shards (all ranks must agree; bfloat16 is what the kernel writes).
    Returns {module index: tensor} with every module, on `device`.  One all_gather per round; ranks that
    have run out of modules contribute zeros.
    """
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    if sorted(local) != plan[rank]:
        raise ValueError(f"rank {rank} holds modules {sorted(local)} but the plan assigns {plan[rank]}")
    some = next(iter(local.values())) if local else None
    if device is None:
        if some is not None:
            device = some.device
        elif dist.get_backend(group) == "nccl":
            device = torch.device("cuda", torch.cuda.current_device())
        else:
            device = torch.device("cpu")
    if some is not None and some.dtype != dtype:
        raise ValueError(f"local shards are {some.dtype}, the exchange was asked for {dtype}")
    out = dict(local)
    for rnd in range(max(len(p) for p in plan)):
        idx = [p[rnd] if rnd < len(p) else None for p in plan]
        numel = max((shapes[i][0] * shapes[i][1] for i in idx if i is not None), default=0)
        send = torch.zeros(numel, dtype=dtype, device=device)
        mine = idx[rank]
        if mine is not None:
            send[: local[mine].numel()] = local[mine].reshape(-1)
        recv = [torch.empty(numel, dtype=dtype, device=device) for _ in range(world)]
        dist.all_gather(recv, send, group=group)
        for r, i in enumerate(idx):
            if i is not None and r != rank:
                d_o, d_i = shapes[i]
                out[i] = recv[r][: d_o * d_i].reshape(d_o, d_i).clone()
    return out
