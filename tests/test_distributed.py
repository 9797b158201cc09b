"""CPU tests of the data-parallel host logic on 2 gloo ranks: shard arithmetic and the
scalar loss all-reduce give the same total as one process over the whole batch.  (The
per-shard losses come from the CPU oracle here; on GPUs they come from the kernels.)"""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from transducer_b200 import distributed as D
from transducer_b200 import workloads


def test_shard_ranges_cover_batch():
    for batch in (0, 1, 7, 32, 33):
        for world in (1, 2, 3, 8):
            spans = [D.shard_range(batch, r, world) for r in range(world)]
            assert spans[0][0] == 0 and sum(c for _, c in spans) == batch
            for (f0, c0), (f1, _) in zip(spans, spans[1:]):
                assert f0 + c0 == f1
            assert max(c for _, c in spans) - min(c for _, c in spans) <= 1
    with pytest.raises(ValueError):
        D.shard_range(4, 2, 2)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, out):
    from oracle import oracle as O
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    w = workloads.Workload("dp_test", B=5, T=40, U=8, V=24, t_range=(20, 40), u_range=(1, 8))
    first, count = D.shard_range(w.B, rank, world)
    E, P, labels, il, ll = [t.numpy() for t in workloads.generate(w, "cpu", first=first, count=count)]
    costs = O.loss_and_grads(E, P, labels, il, ll, want_grads=False)["costs"]
    local = torch.tensor([float(costs.sum())])
    total = D.all_reduce_loss(local.clone())
    mean = D.mean_loss(local, w.B)
    out[rank] = (float(local), float(total), float(mean))
    dist.destroy_process_group()


def test_two_rank_loss_sum_matches_single_process():
    from oracle import oracle as O
    world = 2
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), out), nprocs=world, join=True)
    w = workloads.Workload("dp_test", B=5, T=40, U=8, V=24, t_range=(20, 40), u_range=(1, 8))
    E, P, labels, il, ll = [t.numpy() for t in workloads.generate(w, "cpu")]
    want = float(O.loss_and_grads(E, P, labels, il, ll, want_grads=False)["costs"].sum())
    assert np.isclose(out[0][1], want, rtol=1e-6) and np.isclose(out[1][1], want, rtol=1e-6)
    assert np.isclose(out[0][0] + out[1][0], want, rtol=1e-6)
    assert np.isclose(out[0][2], want / w.B, rtol=1e-6)


def test_workload_shards_regenerate_identically():
    w = workloads.CONFIGS["c1"]
    full = workloads.generate(w, "cpu")
    part = workloads.generate(w, "cpu", first=1, count=1)
    for a, b in zip(full, part):
        assert torch.equal(a[1:2], b)
