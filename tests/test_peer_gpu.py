"""Peer exchange of the sequence-sharded driver: copy-engine copies into peers' buffers + flag words (GPU)."""
import ctypes as C
import os
import sys

import numpy as np
import pytest
import torch

from tests import gpu_util as gu  # noqa: F401  (sets the path up)

pytestmark = pytest.mark.gpu

import triebwerk_b200 as tq  # noqa: E402


def test_flag_words_and_bounded_wait_on_one_gpu():
    """One process plays both sides on its own buffer: a copy, the flag store behind it, a wait that is satisfied, and a
    wait for a step nobody announces, which must give up after its time limit with status 4 and leave the context
    usable."""
    L = tq.lib()
    ptr, handle = C.c_void_p(), C.create_string_buffer(64)
    nbytes = 256 + 4096 + 256
    assert L.tq_peer_buffer_create(nbytes, C.byref(ptr), handle) == 0
    base = int(ptr.value)
    try:
        src = torch.arange(2048, dtype=torch.float16, device="cuda")
        stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
        assert L.tq_peer_copy(base + 256, src.data_ptr(), 4096, stream) == 0
        flags = (C.c_void_p * 1)(C.c_void_p(base))
        assert L.tq_peer_signal(flags, 1, 3, 7, stream) == 0   # flag word 3 := 7
        assert L.tq_peer_wait(base + 3 * 8, 1, 7, base + 256 + 4096, 1000, stream) == 0
        torch.cuda.synchronize()
        from triebwerk_b200.sharded import _DeviceArray
        data = torch.as_tensor(_DeviceArray(base + 256, (2048,), "<f2"), device="cuda")
        assert torch.equal(data, src)
        status = torch.as_tensor(_DeviceArray(base + 256 + 4096, (1,), "<i4"), device="cuda")
        assert int(status.cpu()[0]) == 0
        # nobody will ever write 8 into word 3: the wait must end by itself
        assert L.tq_peer_wait(base + 3 * 8, 1, 8, base + 256 + 4096, 50, stream) == 0
        torch.cuda.synchronize()
        assert int(status.cpu()[0]) == 4
        assert torch.equal(data, src)  # the context is alive
        # argument checks
        assert L.tq_peer_wait(base, 0, 1, None, 50, stream) != 0
        assert L.tq_peer_wait(base, 1, 1, None, 0, stream) != 0
        assert L.tq_peer_signal(flags, 1, 99, 1, stream) != 0
    finally:
        torch.cuda.synchronize()
        assert L.tq_peer_buffer_destroy(ptr) == 0


def _peer_worker(rank, world, port, q):
    import torch.distributed as dist
    from triebwerk_b200 import sharded
    torch.cuda.set_device(rank)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        lengths = [5, 9, 3, 7, 11]
        plan = sharded.shard_plan(lengths, world)   # ragged: shards of different sizes
        n_layers, row = 6, (48,)
        groups = sharded.layer_groups(n_layers, 3)
        gen = torch.Generator(device="cuda").manual_seed(7)
        full = torch.randn(n_layers, len(lengths), *row, generator=gen, device="cuda").to(torch.float16)  # same on all ranks
        mine = torch.as_tensor(plan[rank], device="cuda", dtype=torch.long)
        a = sharded.PeerCopyGatherer(plan, groups, row)
        b = sharded.LayerGroupGatherer(plan, groups)
        ok = True
        for step in range(3):
            local = (full[:, mine] + step).contiguous()
            for gi, (l0, l1) in enumerate(groups):
                a.gather(gi, local[l0:l1].contiguous())
                b.gather(gi, local[l0:l1].contiguous())
            a.finish()
            b.finish()
            torch.cuda.synchronize()
            ok = ok and torch.equal(a.result(), full + step) and torch.equal(b.result(), full + step)
            dist.barrier()   # nobody starts the next step's copies before everybody has read this one
        ok = ok and a.status() == 0
        a.close()
        q.put((rank, bool(ok)))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_peer_copy_gather_equals_nccl_gather_on_two_gpus():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29600 + os.getpid() % 200
    procs = [ctx.Process(target=_peer_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(180)
    for p in procs:
        if p.is_alive():
            p.kill()   # exactly the child started above
            pytest.fail("a rank did not finish")
        assert p.exitcode == 0
    got = dict(q.get(timeout=5) for _ in procs)
    assert got == {0: True, 1: True}
