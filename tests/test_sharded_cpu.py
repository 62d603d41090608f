"""The N>1 host path on CPU: two gloo ranks shard a ragged batch, each computes its sequences (with the CPU
oracle standing in for the GPU kernels -- this test is about the sharding and the gather), outputs are
gathered and must equal the single-process result."""
import os
import socket
import sys

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _problem():
    from oracle import tqo
    from tests import helpers as hp
    rng = np.random.default_rng(11)
    R, _ = tqo.rotation()
    H, Hkv, D, msl, bits = 8, 4, 128, 64, 4
    lengths = [64, 3, 40, 17, 5, 60, 33]
    ck, kn, cv, vn = hp.build_cache_oracle(rng, len(lengths), lengths, msl, Hkv, D, bits, R)
    q = rng.standard_normal((len(lengths), H * D)).astype(np.float16)
    return dict(R=R, H=H, Hkv=Hkv, D=D, msl=msl, bits=bits, lengths=lengths, ck=ck, kn=kn, cv=cv, vn=vn, q=q)


def _attend(pb, ids):
    from oracle import tqo
    msl = pb["msl"]
    rows = np.concatenate([np.arange(g * msl, (g + 1) * msl) for g in ids]) if ids else np.zeros(0, np.int64)
    pos = np.array([pb["lengths"][g] - 1 for g in ids], np.int32)
    if not ids:
        return np.zeros((0, pb["H"] * pb["D"]), np.float16)
    out, _ = tqo.attention_batch(pb["q"][ids], pb["ck"][rows], pb["cv"][rows], pb["kn"][rows], pb["vn"][rows], pb["R"],
                                 pos, msl, pb["H"], pb["Hkv"], pb["D"], pb["bits"])
    return out


def _worker(rank, world, port, ret):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from triebwerk_b200.sharded import gather_outputs, shard_plan
        pb = _problem()
        plan = shard_plan(pb["lengths"], world)
        local = torch.from_numpy(_attend(pb, plan[rank]))
        full = gather_outputs(local, plan)
        ret[rank] = (plan, full.numpy().copy())
    finally:
        dist.destroy_process_group()


def test_two_ranks_reproduce_single_process_result():
    world = 2
    port = _free_port()
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, port, ret), nprocs=world, join=True)
    pb = _problem()
    ref = _attend(pb, list(range(len(pb["lengths"]))))
    plan0, out0 = ret[0]
    plan1, out1 = ret[1]
    assert plan0 == plan1
    assert sorted(i for p in plan0 for i in p) == list(range(len(pb["lengths"])))
    loads = [sum(pb["lengths"][i] for i in p) for p in plan0]
    assert abs(loads[0] - loads[1]) <= max(pb["lengths"])
    assert (out0.view(np.uint16) == ref.view(np.uint16)).all()
    assert (out1.view(np.uint16) == ref.view(np.uint16)).all()


def _worker_groups(rank, world, port, ret):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from triebwerk_b200.sharded import LayerGroupGatherer, layer_groups, shard_plan
        lengths = [9, 3, 40, 17, 5, 60, 33]
        plan = shard_plan(lengths, world)
        n_layers, width = 5, 6
        groups = layer_groups(n_layers, 3)
        assert groups[0][0] == 0 and groups[-1] == (n_layers - 1, n_layers)
        assert all(a[1] == b[0] for a, b in zip(groups, groups[1:]))
        # value of (layer, sequence, column) is unique, so misplaced rows show
        full = torch.arange(n_layers * len(lengths) * width, dtype=torch.float32).view(n_layers, len(lengths), width)
        local = full[:, plan[rank]].contiguous()
        gat = LayerGroupGatherer(plan, groups)
        for step in range(2):  # buffers are reused from step to step
            for gi, (l0, l1) in enumerate(groups):
                gat.gather(gi, local[l0:l1] + step)
            gat.finish()
            ret[(rank, step)] = gat.result().numpy().copy()
    finally:
        dist.destroy_process_group()


def test_layer_group_gather_two_ranks():
    world = 2
    port = _free_port()
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker_groups, args=(world, port, ret), nprocs=world, join=True)
    ref = np.arange(5 * 7 * 6, dtype=np.float32).reshape(5, 7, 6)
    for rank in range(world):
        for step in range(2):
            assert (ret[(rank, step)] == ref + step).all()
