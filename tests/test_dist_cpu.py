"""Host-side logic of the multi-GPU forms, run as two gloo ranks on CPU."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from jax_gptq_b200 import dist as D
from oracle import ref_gptq as R


def test_shard_range_covers_everything():
    for total, world, mult in [(3072, 8, 16), (909, 4, 1), (50257, 8, 16), (16, 8, 16), (0, 2, 1)]:
        got = [D.shard_range(total, r, world, mult) for r in range(world)]
        assert got[0][0] == 0 and got[-1][1] == total
        for (b0, e0), (b1, e1) in zip(got, got[1:]):
            assert e0 == b1 and b0 <= e0
        assert all(b % mult == 0 for b, _ in got)
    with pytest.raises(ValueError):
        D.shard_range(10, 3, 2)


def test_assign_layers_balances():
    costs = [8, 1, 1, 1, 1, 1, 1, 1, 1, 8]
    owner = D.assign_layers(costs, 2)
    loads = [sum(c for c, o in zip(costs, owner) if o == r) for r in range(2)]
    assert sorted(loads) == [12, 12] and len(owner) == len(costs)


def _free_port():
    with socket.socket() as s:
        s.bind(('127.0.0.1', 0))
        return s.getsockname()[1]


def _worker(rank, world, port, q):
    os.environ['MASTER_ADDR'] = '127.0.0.1'
    os.environ['MASTER_PORT'] = str(port)
    dist.init_process_group('gloo', rank=rank, world_size=world)
    try:
        rng = np.random.default_rng(5)
        X = rng.standard_normal((96, 24)).astype(np.float32)          # same on every rank
        b, e = D.shard_range(X.shape[0], rank, world)
        local = X[b:e]
        H_sum = torch.from_numpy(local.T @ local)
        H_sum, n = D.allreduce_hessian(H_sum, local.shape[0])
        H = (H_sum / n).numpy()
        ref = R.accumulate_H_direct([X])
        ok_h = bool(np.allclose(H, ref, atol=1e-6)) and n == 96
        # column slabs of a product, gathered back
        W = rng.standard_normal((24, 10)).astype(np.float32)
        c0, c1 = D.shard_range(10, rank, world)
        slab = torch.from_numpy(X @ W[:, c0:c1])
        full = D.gather_columns(slab, (c0, c1), 10).numpy()
        ok_g = bool(np.allclose(full, X @ W, atol=1e-5))
        q.put((rank, ok_h, ok_g))
    finally:
        dist.destroy_process_group()


def test_allreduce_and_gather_two_ranks():
    world = 2
    ctx = mp.get_context('spawn')
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert sorted(r[0] for r in results) == [0, 1]
    assert all(r[1] and r[2] for r in results)
