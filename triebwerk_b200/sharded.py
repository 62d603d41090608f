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


class LayerGroupGatherer:
    """Gathers the outputs of a decode step one GROUP OF LAYERS at a time, on a side stream, while the next group is
    being computed: only the last group's exchange is left exposed at the end of the step.

    Usage per step: for every group ``gather(group_index, local_out[l0:l1])`` right after the group's kernels were
    enqueued, then ``finish()`` (the compute stream waits for the exchanges).  ``result()`` assembles
    ``[layers, n_total, ...]`` in global sequence order.  On CPU tensors (gloo) everything runs inline.
    """

    def __init__(self, plan: List[List[int]], layer_groups: Sequence[Sequence[int]], group=None):
        self.plan, self.group = plan, group
        self.layer_groups = [(int(a), int(b)) for a, b in layer_groups]  # [first, end) per group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.n_max = max(len(p) for p in plan)
        self.n_total = sum(len(p) for p in plan)
        self._bufs = {}
        self._stream = None
        self._events = []

    def _buffers(self, gi: int, like: torch.Tensor):
        key = (gi, tuple(like.shape[2:]), like.dtype, like.device)
        if key not in self._bufs:
            l0, l1 = self.layer_groups[gi]
            shape = (l1 - l0, self.n_max) + tuple(like.shape[2:])
            pad = torch.zeros(shape, dtype=like.dtype, device=like.device)
            out = torch.empty((self.world,) + shape, dtype=like.dtype, device=like.device)
            self._bufs[key] = (pad, out)
        return self._bufs[key]

    def gather(self, gi: int, local_out: torch.Tensor) -> None:
        """local_out: [layers of group gi, n_local, ...] for the sequences plan[rank]."""
        l0, l1 = self.layer_groups[gi]
        n_local = len(self.plan[self.rank])
        assert local_out.shape[0] == l1 - l0 and local_out.shape[1] == n_local
        pad, out = self._buffers(gi, local_out)
        src = local_out
        if local_out.is_cuda:
            if self._stream is None:
                self._stream = torch.cuda.Stream(device=local_out.device)
            ev = torch.cuda.Event()
            ev.record(torch.cuda.current_stream(local_out.device))
            with torch.cuda.stream(self._stream):
                self._stream.wait_event(ev)
                if n_local != self.n_max:
                    pad[:, :n_local].copy_(local_out)
                    src = pad
                dist.all_gather_into_tensor(out.view((-1,) + tuple(out.shape[2:])), src.contiguous(), group=self.group)
                done = torch.cuda.Event()
                done.record(self._stream)
            self._events.append(done)
        else:
            if n_local != self.n_max:
                pad[:, :n_local].copy_(local_out)
                src = pad
            dist.all_gather_into_tensor(out.view((-1,) + tuple(out.shape[2:])), src.contiguous(), group=self.group)

    def finish(self) -> None:
        """The current stream waits for every exchange issued since the last finish()."""
        for ev in self._events:
            torch.cuda.current_stream().wait_event(ev)
        self._events = []

    def result(self) -> torch.Tensor:
        """[layers, n_total, ...] in global sequence order, from the groups gathered last."""
        parts = []
        for gi, (l0, l1) in enumerate(self.layer_groups):
            key = next(k for k in self._bufs if k[0] == gi)
            _, out = self._bufs[key]
            full = torch.empty((l1 - l0, self.n_total) + tuple(out.shape[3:]), dtype=out.dtype, device=out.device)
            for r, ids in enumerate(self.plan):
                if ids:
                    idx = torch.as_tensor(ids, device=out.device, dtype=torch.long)
                    full.index_copy_(1, idx, out[r, :, : len(ids)])
            parts.append(full)
        return torch.cat(parts, 0)


def layer_groups(n_layers: int, n_groups: int = 4) -> List[tuple]:
    """[first, end) layer ranges for LayerGroupGatherer: about equal groups, the last one a single layer (its exchange
    is the only one nothing hides)."""
    if n_layers <= 2 or n_groups <= 1:
        return [(0, n_layers)]
    n_groups = min(n_groups, n_layers)
    body = n_layers - 1
    cuts = [round(i * body / (n_groups - 1)) for i in range(n_groups)]
    groups = [(cuts[i], cuts[i + 1]) for i in range(n_groups - 1) if cuts[i + 1] > cuts[i]]
    return groups + [(body, n_layers)]
