"""Multi-GPU forms of the hot path: one process per GPU, `torch.distributed` for the plumbing.

The reference is single-GPU (quantize_interpreter.py:116-117 pins ``gpu[0]``); these are the
three shardings the path offers, none of which changes a result beyond fp32 summation order:

* calibration tokens sharded over ranks: every rank accumulates X^T X of its own tokens, one
  all-reduce (NCCL over NVLink on GPUs) of the K x K sums and of the sample count gives every
  rank the full Hessian (`allreduce_hessian`, `gptq_token_sharded`);
* output channels are independent given the Hessian (gptq.py:136-147 only couples rows), so
  each rank quantizes its own slab of columns (`gptq_token_sharded(..., shard_columns=True)`);
* the packed matmul is sharded over output channels, activations replicated, no collective for
  the product itself; an all-gather assembles the full output when asked
  (`quantized_matmul_column_sharded`).
* independent layers go to different ranks (`assign_layers`).

Functions that only move data or plan shards work on CPU tensors with the gloo backend too,
which is how the host-side logic is tested without GPUs.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def _world(group=None):
    if not dist.is_available() or not dist.is_initialized():
        return 0, 1
    return dist.get_rank(group), dist.get_world_size(group)


def shard_range(total, rank, world, multiple=1):
    """[begin, end) of shard `rank` when `total` items are split into `world` contiguous shards whose
    boundaries are multiples of `multiple` (the last shard takes the remainder)."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError(f'bad rank {rank} / world {world}')
    units = -(-total // multiple)
    b = (units * rank // world) * multiple
    e = (units * (rank + 1) // world) * multiple
    return min(b, total), min(e, total)


def assign_layers(costs, world):
    """Greedy longest-processing-time assignment of independent layers to ranks.
    `costs[i]` is the work of layer i (e.g. K*K*n + K*K*K); returns a list of rank ids."""
    order = sorted(range(len(costs)), key=lambda i: -costs[i])
    load = [0.0] * world
    owner = [0] * len(costs)
    for i in order:
        r = min(range(world), key=lambda j: (load[j], j))
        owner[i] = r
        load[r] += costs[i]
    return owner


def allreduce_hessian(H_sum, n_local, group=None):
    """Sum the per-rank raw second-moment sums (K x K, fp32) and sample counts over the group.
    Returns (H_sum_global, n_global); H_sum is reduced in place."""
    rank, world = _world(group)
    if world == 1:
        return H_sum, int(n_local)
    n = torch.tensor([float(n_local)], dtype=torch.float64, device=H_sum.device)
    dist.all_reduce(H_sum, op=dist.ReduceOp.SUM, group=group)
    dist.all_reduce(n, op=dist.ReduceOp.SUM, group=group)
    return H_sum, int(round(float(n.item())))


def gptq_token_sharded(W, xs_local, block_size=128, actorder=False, damping=0.01, bits=4, group=None,
                       shard_columns=True, multiple=16):
    """GPTQ of one linear with the calibration tokens sharded over the ranks of `group`.

    Every rank passes the full W (K x N) and ITS OWN batches.  The Hessian is all-reduced; with
    `shard_columns` each rank then quantizes only columns shard_range(N, rank, world, multiple)
    and gets (Q_slab, params_slab, (c0, c1)); otherwise every rank quantizes all columns.
    """
    from . import gptq as G
    rank, world = _world(group)
    Wd = G._to_dev(W)
    status = torch.zeros(1, dtype=torch.int32, device=Wd.device)
    H_sum, n_local = G._accumulate_raw(xs_local, status=status)
    H_sum, n = allreduce_hessian(H_sum, n_local, group)
    H = G._finalize_H(H_sum, n)
    G._raise_status(int(status.item()) << 8)
    c0, c1 = (0, Wd.shape[1])
    if shard_columns and world > 1:
        c0, c1 = shard_range(Wd.shape[1], rank, world, multiple)
    Wslab = Wd[:, c0:c1].contiguous()
    if c1 == c0:
        return None, None, (c0, c1)
    Q, params = G.gptq(Wslab, None, block_size=block_size, actorder=actorder, damping=damping, bits=bits, H=H)
    return Q, params, (c0, c1)


def gather_columns(slab, col_range, N, group=None):
    """All-gather column slabs (rows x (c1-c0)) of a (rows x N) matrix; every rank gets the whole."""
    rank, world = _world(group)
    if world == 1:
        return slab
    rows = slab.shape[0]
    sizes = torch.zeros(world, dtype=torch.int64, device=slab.device)
    sizes[rank] = slab.shape[1]
    dist.all_reduce(sizes, group=group)
    sizes = [int(v) for v in sizes.tolist()]
    wmax = max(sizes)
    buf = torch.zeros((rows, wmax), dtype=slab.dtype, device=slab.device)
    buf[:, :slab.shape[1]] = slab
    outs = [torch.empty_like(buf) for _ in range(world)]
    dist.all_gather(outs, buf, group=group)
    return torch.cat([o[:, :w] for o, w in zip(outs, sizes)], dim=1)


def quantized_matmul_column_sharded(x, qm_shard, group=None, gather=True, N=None):
    """x (replicated) @ dequant(this rank's column shard).  With `gather`, returns the full (.., N)
    product on every rank; otherwise the local (.., N_local) slab."""
    from .op import quantized_matmul
    y = quantized_matmul(x, qm_shard)
    rank, world = _world(group)
    if not gather or world == 1:
        return y
    lead = y.shape[:-1]
    y2 = y.reshape(-1, y.shape[-1])
    full = gather_columns(y2, None, N if N is not None else -1, group)
    return full.reshape(tuple(lead) + (full.shape[-1],))
