"""Multi-GPU driver of the path: one process per GPU, whole sequences per rank, one gather of outputs.

No kernel reads another GPU's memory and no cache byte crosses NVLink.  The only exchange is the final
gather of the per-sequence attention outputs ([n_local, ...] fp16), done with ``torch.distributed``
(NCCL on GPUs, gloo in the CPU tests).  Ragged shard sizes are handled by padding to the largest shard.
"""
from __future__ import annotations

from typing import List, Sequence

import torch
import torch.distributed as dist

from .partition import contiguous_partition, lpt_partition


def shard_plan(lengths: Sequence[int], world: int, balance: str = "auto") -> List[List[int]]:
    """Sequence ids per rank.  Equal lengths -> contiguous blocks; otherwise LPT by tokens."""
    if balance == "contiguous" or (balance == "auto" and len(set(int(x) for x in lengths)) <= 1):
        return contiguous_partition(len(lengths), world)
    return lpt_partition(lengths, world)


def gather_outputs(local_out: torch.Tensor, plan: List[List[int]], group=None) -> torch.Tensor:
    """All ranks get the outputs of all sequences in global sequence order.

    local_out: [n_local, ...] for the sequences plan[rank] (in that order).  Returns [n_total, ...].
    """
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    assert local_out.shape[0] == len(plan[rank]), "local outputs do not match the shard plan"
    n_max = max(len(p) for p in plan)
    n_total = sum(len(p) for p in plan)
    pad = torch.zeros((n_max,) + tuple(local_out.shape[1:]), dtype=local_out.dtype, device=local_out.device)
    pad[: local_out.shape[0]] = local_out
    gathered = torch.empty((world * n_max,) + tuple(local_out.shape[1:]), dtype=local_out.dtype,
                           device=local_out.device)
    dist.all_gather_into_tensor(gathered, pad, group=group)
    out = torch.empty((n_total,) + tuple(local_out.shape[1:]), dtype=local_out.dtype, device=local_out.device)
    for r, ids in enumerate(plan):
        if ids:
            idx = torch.as_tensor(ids, device=local_out.device, dtype=torch.long)
            out.index_copy_(0, idx, gathered[r * n_max: r * n_max + len(ids)])
    return out
