"""Two-GPU check of the sharded forms (skipped on boxes with one GPU): token-sharded Hessian +
NCCL all-reduce + column-sharded quantization against the single-GPU result, and the
column-sharded packed matmul against the unsharded one."""
import os
import socket

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(('127.0.0.1', 0))
        return s.getsockname()[1]


def _worker(rank, world, port, q):
    import torch.distributed as dist
    import importlib
    os.environ['MASTER_ADDR'] = '127.0.0.1'
    os.environ['MASTER_PORT'] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group('nccl', rank=rank, world_size=world, device_id=torch.device('cuda', rank))
    try:
        G = importlib.import_module('jax_gptq_b200.gptq')
        D = importlib.import_module('jax_gptq_b200.dist')
        op = importlib.import_module('jax_gptq_b200.op')
        rng = np.random.default_rng(77)
        K, N, n = 512, 640, 4096
        W = torch.from_numpy((0.02 * rng.standard_normal((K, N))).astype(np.float32)).cuda()
        X = torch.from_numpy(rng.standard_normal((n, K)).astype(np.float32)).cuda()
        b, e = D.shard_range(n, rank, world)
        Q, params, (c0, c1) = D.gptq_token_sharded(W, [X[b:e]], block_size=128)
        Q_full, p_full = G.gptq(W, [X], block_size=128)
        same = float((Q == Q_full[:, c0:c1]).float().mean().item())
        ok_scale = bool(torch.equal(params['scale'], p_full['scale'][c0:c1]))
        # column-sharded matmul
        qm_full = G.pack_matrix(Q_full, p_full)
        qm_shard = G.pack_matrix(Q_full[:, c0:c1].contiguous(),
                                 {'scale': p_full['scale'][c0:c1].contiguous(), 'zero': p_full['zero'][c0:c1].contiguous(),
                                  'maxq': 15})
        x = X[:16].half()
        y_full = op.quantized_matmul(x, qm_full)
        y = D.quantized_matmul_column_sharded(x, qm_shard, gather=True, N=N)
        err = float((y.float() - y_full.float()).abs().max().item())
        # the whole layer loop on the ranks: lower-triangle all-reduce, column-sharded quantize, all-gather
        jobs = [(W, [X[b:e]]), (W[:, :320].contiguous(), [X[b:e]])]
        ref0 = G.pack_matrix(Q_full, p_full).int_weight
        same_pipe, ok_pipe = 1.0, True
        for mode in ('owner', 'columns'):        # reduce to an owner rank + broadcast; all-reduce + column slabs + all-gather
            pipe = D.ShardedPipeline(streams=2, mode=mode)
            res = pipe.run(jobs, n, block_size=128)
            torch.cuda.synchronize()
            same_pipe = min(same_pipe, float((res[0][0] == ref0).float().mean().item()))
            ok_pipe = ok_pipe and tuple(res[0][0].shape) == (K // 2, N) and tuple(res[1][0].shape) == (K // 2, 320) \
                and bool(torch.equal(res[0][1], p_full['scale']))
        # linears (not tokens) sharded: every linear entirely on its owner, from all tokens - the single-GPU bytes
        pipe = D.ShardedPipeline(streams=2, mode='layers')
        jobs_full = [(W, [X]), (W[:, :320].contiguous(), [X]), (W[:, 320:].contiguous(), [X])]
        res = pipe.run(jobs_full, n, block_size=128)
        torch.cuda.synchronize()
        Q1, p1 = G.gptq(jobs_full[2][0], [X], block_size=128)
        ok_pipe = ok_pipe and bool(torch.equal(res[0][0], ref0)) and bool(torch.equal(res[0][1], p_full['scale'])) \
            and bool(torch.equal(res[2][0], G.pack_matrix(Q1, p1).int_weight)) and tuple(res[1][0].shape) == (K // 2, 320)
        q.put((rank, same, ok_scale, err, tuple(y.shape), same_pipe, ok_pipe))
    finally:
        dist.destroy_process_group()


def test_token_and_column_sharding_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip('needs two GPUs')
    import torch.multiprocessing as mp
    world = 2
    ctx = mp.get_context('spawn')
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=150) for _ in range(world)]
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    for rank, same, ok_scale, err, shape, same_pipe, ok_pipe in results:
        assert same >= 0.999, f'rank {rank}: identical values {same}'
        assert ok_scale
        assert err <= 2e-2 and shape == (16, 640)
        assert same_pipe >= 0.998 and ok_pipe, f'rank {rank}: pipeline bytes identical {same_pipe}'


def test_lower_triangle_pack_roundtrip():
    """What the all-reduce sends: the tiles on or below the diagonal, packed and unpacked without loss."""
    import importlib
    D = importlib.import_module('jax_gptq_b200.dist')
    from jax_gptq_b200 import _lib
    for K in (128, 256, 768, 840, 1000):
        H = torch.randn(K, K, device='cuda')
        P = D.pack_lower(H)
        assert P.numel() == _lib.lib.jgq_hessian_lower_elems(K)
        H2 = torch.full((K, K), float('nan'), device='cuda')
        D.unpack_lower(P, H2)
        i = torch.arange(K, device='cuda')
        keep = i[None, :] < (128 * (i // 128 + 1))[:, None]
        assert torch.equal(H2[keep], H[keep])
        assert bool(torch.isnan(H2[~keep]).all())
        assert bool(keep[i[:, None] >= i[None, :]].all())          # the lower triangle is inside what travels
