"""Multi-GPU driver of the path: one process per GPU, whole sequences per rank, one gather of outputs.

No kernel reads another GPU's memory and no cache byte crosses NVLink.  The only exchange is the
gather of the per-sequence attention outputs ([n_local, ...] fp16): with ``torch.distributed`` (NCCL on GPUs, gloo in
the CPU tests; LayerGroupGatherer), or -- on GPUs of one node -- with copy-engine copies straight into every peer's
buffer (PeerCopyGatherer), which take no SM from the attention kernel.  Ragged shard sizes are handled by padding to
the largest shard.
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


class _DeviceArray:
    """A device allocation that is not torch's, shown to torch through the CUDA array interface."""

    def __init__(self, ptr: int, shape, typestr: str):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr, "data": (int(ptr), False), "version": 3}


class PeerCopyGatherer:
    """The interface of LayerGroupGatherer with the exchange done by the copy engines.

    Every rank owns one buffer ``[flags | world x layers x n_max x row]`` whose CUDA IPC handle its peers open once.
    ``gather(gi, local_out[l0:l1])`` enqueues, on a side stream behind the group's kernels, one device-to-device copy
    per peer (and one into the own buffer) of the group's rows into slice ``rank`` of that peer's buffer; copy engines
    move them over NVLink while the SMs work on the next group.  ``finish()`` writes the step number into every peer's
    flag word ``rank`` behind the copies, and makes the compute stream wait until all ``world`` flag words of the own
    buffer carry it (a kernel with a time limit; on expiry it raises ``status()`` and returns).  A rank may start the
    copies of its next step only after its peers are done reading the previous one: callers that consume ``result()``
    separate steps by a barrier, as the collectives they replace did implicitly.
    """

    FLAG_BYTES = 256  # TQ_PEER_MAX 8-byte words

    def __init__(self, plan: List[List[int]], layer_groups: Sequence[Sequence[int]], row_shape, dtype=torch.float16,
                 group=None, wait_limit_ms: int = 2000):
        import ctypes as C
        from ._lib import lib
        self._C, self._lib = C, lib()
        self.plan, self.group = plan, group
        self.layer_groups = [(int(a), int(b)) for a, b in layer_groups]
        self.n_layers = max(b for _, b in self.layer_groups)
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        assert self.world <= 32
        self.n_max = max(len(p) for p in plan)
        self.n_total = sum(len(p) for p in plan)
        self.row_shape = tuple(int(x) for x in row_shape)
        self.dtype = dtype
        self.itemsize = torch.empty((), dtype=dtype).element_size()
        self.row_elems = 1
        for x in self.row_shape:
            self.row_elems *= x
        self.row_bytes = self.row_elems * self.itemsize
        self.slice_bytes = self.n_layers * self.n_max * self.row_bytes      # one source rank's part of a buffer
        self.bytes = self.FLAG_BYTES + self.world * self.slice_bytes + 256   # + the status word
        self.status_off = self.FLAG_BYTES + self.world * self.slice_bytes
        self.limit_ms = int(wait_limit_ms)
        self.step = 0
        # Set-up is collective: a rank whose allocation or mapping fails still takes part in the exchange of handles and
        # in the agreement that follows, so that all ranks raise together instead of some of them waiting forever.
        ptr, handle = C.c_void_p(), C.create_string_buffer(64)
        err = None
        r = self._lib.tq_peer_buffer_create(self.bytes, C.byref(ptr), handle)
        if r != 0:
            err = f"tq_peer_buffer_create failed ({r})"
        self.own = int(ptr.value or 0)
        handles = [None] * self.world
        dist.all_gather_object(handles, bytes(handle.raw) if err is None else None, group=group)
        self.peers = []
        for r_, h in enumerate(handles):
            if r_ == self.rank or h is None or err is not None:
                self.peers.append(self.own if r_ == self.rank else 0)
                if h is None and err is None:
                    err = f"rank {r_} has no buffer"
                continue
            q = C.c_void_p()
            rc = self._lib.tq_peer_buffer_open(C.create_string_buffer(h, 64), C.byref(q))
            if rc != 0:
                err = f"tq_peer_buffer_open of rank {r_}'s buffer failed ({rc})"
            self.peers.append(int(q.value or 0))
        oks = [None] * self.world
        dist.all_gather_object(oks, err, group=group)
        bad = [f"rank {i}: {e}" for i, e in enumerate(oks) if e is not None]
        if bad:
            self._release()
            raise RuntimeError("peer buffers could not be set up: " + "; ".join(bad))
        typestr = {torch.float16: "<f2", torch.float32: "<f4", torch.bfloat16: "<u2"}[dtype]
        view = torch.as_tensor(_DeviceArray(self.own + self.FLAG_BYTES, (self.world, self.n_layers, self.n_max) + self.row_shape,
                                            typestr), device="cuda")
        self._data = view if dtype != torch.bfloat16 else view.view(torch.bfloat16)
        self._stream = torch.cuda.Stream()
        # one stream per peer: the copies to different peers run on different copy engines at the same time
        self._peer_streams = [self._stream if r_ == self.rank else torch.cuda.Stream() for r_ in range(self.world)]
        self._flag_ptrs = (C.c_void_p * self.world)(*[C.c_void_p(p) for p in self.peers])

    def gather(self, gi: int, local_out: torch.Tensor) -> None:
        """local_out: [layers of group gi, n_local, ...] for the sequences plan[rank]."""
        l0, l1 = self.layer_groups[gi]
        n_local = len(self.plan[self.rank])
        assert local_out.is_cuda and local_out.dtype == self.dtype and local_out.is_contiguous()
        assert local_out.shape[0] == l1 - l0 and local_out.shape[1] == n_local and tuple(local_out.shape[2:]) == self.row_shape
        ev = torch.cuda.Event()
        ev.record(torch.cuda.current_stream())
        base = self.FLAG_BYTES + self.rank * self.slice_bytes
        for k in range(self.world):
            r_ = (self.rank + 1 + k) % self.world  # every rank starts with another peer
            peer, s = self.peers[r_], self._peer_streams[r_]
            s.wait_event(ev)
            sp = self._C.c_void_p(s.cuda_stream)
            if n_local == self.n_max:   # the group's layers are one contiguous run on both sides
                rc = self._lib.tq_peer_copy(peer + base + l0 * self.n_max * self.row_bytes, local_out.data_ptr(),
                                            (l1 - l0) * self.n_max * self.row_bytes, sp)
                if rc != 0:
                    raise RuntimeError(f"tq_peer_copy failed ({rc})")
            else:
                for l in range(l0, l1):
                    rc = self._lib.tq_peer_copy(peer + base + l * self.n_max * self.row_bytes,
                                                local_out.data_ptr() + (l - l0) * n_local * self.row_bytes,
                                                n_local * self.row_bytes, sp)
                    if rc != 0:
                        raise RuntimeError(f"tq_peer_copy failed ({rc})")
            local_out.record_stream(s)

    def finish(self) -> None:
        """Announce this rank's copies of the step to every peer; the current stream waits for all peers' copies."""
        self.step += 1
        for r_, s in enumerate(self._peer_streams):
            if r_ != self.rank:
                e = torch.cuda.Event()
                e.record(s)
                self._stream.wait_event(e)
        sp = self._C.c_void_p(self._stream.cuda_stream)
        rc = self._lib.tq_peer_signal(self._flag_ptrs, self.world, self.rank, self.step, sp)
        if rc == 0:
            rc = self._lib.tq_peer_wait(self.own, self.world, self.step, self.own + self.status_off, self.limit_ms, sp)
        if rc != 0:
            raise RuntimeError(f"peer signal / wait failed ({rc})")
        done = torch.cuda.Event()
        done.record(self._stream)
        torch.cuda.current_stream().wait_event(done)

    def status(self) -> int:
        """0, or 4 after a wait for the peers ran out of time."""
        word = torch.as_tensor(_DeviceArray(self.own + self.status_off, (1,), "<i4"), device="cuda")
        return int(word.cpu()[0])

    def result(self) -> torch.Tensor:
        """[layers, n_total, ...] in global sequence order, from the step gathered last."""
        full = torch.empty((self.n_layers, self.n_total) + self.row_shape, dtype=self.dtype, device="cuda")
        for r, ids in enumerate(self.plan):
            if ids:
                idx = torch.as_tensor(ids, device="cuda", dtype=torch.long)
                full.index_copy_(1, idx, self._data[r, :, : len(ids)])
        return full

    def _release(self) -> None:
        for r_, p in enumerate(self.peers):
            if r_ != self.rank and p:
                self._lib.tq_peer_buffer_close(p)
        self.peers = []
        dist.barrier(group=self.group)  # nobody may still copy into a buffer that is about to be freed
        if self.own:
            self._lib.tq_peer_buffer_destroy(self.own)
            self.own = 0

    def close(self) -> None:
        """Unmap the peers' buffers and, after a barrier, free the own one.  Collective."""
        torch.cuda.synchronize()
        self._data = None
        self._release()


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
