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


def _raw_stream():
    return torch._C._cuda_getCurrentRawStream(torch.cuda.current_device())


def pack_lower(H_sum, out=None):
    """The tiles on or below the diagonal of a raw K x K sum (all that carries data before finalize) as one
    contiguous fp32 vector: what has to travel in the all-reduce.  CUDA tensors only."""
    from ._lib import lib, check
    K = H_sum.shape[0]
    n = lib.jgq_hessian_lower_elems(K)
    if out is None:
        out = torch.zeros(n, dtype=torch.float32, device=H_sum.device)
    check(lib.jgq_hessian_pack_lower(H_sum.data_ptr(), K, out.data_ptr(), _raw_stream()))
    return out


def unpack_lower(packed, H_sum):
    from ._lib import lib, check
    K = H_sum.shape[0]
    check(lib.jgq_hessian_unpack_lower(packed.data_ptr(), K, H_sum.data_ptr(), _raw_stream()))
    return H_sum


def allreduce_hessian(H_sum, n_local, group=None, lower_only=True):
    """Sum the per-rank raw second-moment sums (K x K, fp32) and sample counts over the group.
    Returns (H_sum_global, n_global); H_sum is reduced in place.  On CUDA tensors with K % 4 == 0 only the
    tiles on or below the diagonal are sent (about half the bytes); `lower_only=False` sends the square."""
    rank, world = _world(group)
    if world == 1:
        return H_sum, int(n_local)
    n = torch.tensor([float(n_local)], dtype=torch.float64, device=H_sum.device)
    if lower_only and H_sum.is_cuda and H_sum.shape[0] % 4 == 0 and H_sum.is_contiguous():
        packed = pack_lower(H_sum)
        dist.all_reduce(packed, op=dist.ReduceOp.SUM, group=group)
        unpack_lower(packed, H_sum)
    else:
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


class ShardedPipeline:
    """The layer loop for one model on several GPUs: calibration tokens sharded over the ranks, one NCCL
    reduction of the lower triangle of every Hessian, the sequential stages of different linears on
    different ranks, the packed results sent to everybody.

    Per linear, on every rank: Hessian of the local tokens (Hessian stream) -> pack the lower tiles ->
    NCCL reduce to the linear's owner (communication stream, first communicator).  The owner - chosen by a
    greedy longest-job-first assignment that every rank computes identically - unpacks, finalizes with the
    global token count, damps + inverts, quantizes and packs the whole linear on one of its compute streams
    and puts the result into its output buffer, which it broadcasts once, after its last linear (second
    communication stream, second communicator, so that it never holds up a reduction): one collective per
    rank, not one per linear.  The reduction of linear i overlaps the
    Hessian GEMM of linear i+1 and the sequential stages of the linears before it.  Every rank issues the same
    collectives in the same order.

    `mode='columns'` is the other split the path offers: an all-reduce, a replicated inverse on every rank,
    the quantize loop sharded over output channels, an all-gather of the packed slabs.  It has no idle
    ranks for a single linear but repeats the inverse N times; `mode='owner'` divides all the sequential
    work by N as soon as there are several linears.

    `mode='layers'` shards the LINEARS instead of the tokens: every linear is quantized entirely by its
    owner rank (`gptq_many` on the owner's subset, with all of that linear's calibration tokens, which
    every rank passes or at least its owner does), no Hessian travels, and the only collectives are the
    owners' result broadcasts.  For a model of many small linears this is the faster split - a Hessian over
    1/N of the tokens keeps its fixed costs - while a single large linear needs the token split."""

    def __init__(self, streams=6, group=None, mode='owner'):
        self.rank, self.world = _world(group)
        self.mode = mode
        self.group_ar = group
        self.group_ag = dist.new_group() if self.world > 1 else None      # its own NCCL communicator
        self.hstreams = [torch.cuda.Stream(priority=0) for _ in range(2)]     # take turns, like gptq_many's
        self.comm_ar = torch.cuda.Stream(priority=-1)
        self.comm_ag = torch.cuda.Stream(priority=-1)
        self.workers = [torch.cuda.Stream(priority=-1) for _ in range(max(1, streams))]
        self.arenas = None                # one per worker, created on first use (fixed addresses: replayable stages)
        self.nslots = len(self.workers) + 2
        self.bufs = {}
        self.stats = {}

    def _buf(self, tag, shape, dtype, zero=False):
        key = (tag, tuple(shape), dtype)
        t = self.bufs.get(key)
        if t is None:
            t = torch.zeros(tuple(shape), dtype=dtype, device='cuda')
            self.bufs[key] = t
        elif zero:
            t.zero_()
        return t

    def _run_layers(self, jobs, block_size, damping, bits, gather):
        """Linears sharded over the ranks: this rank quantizes the ones it owns, from all their tokens."""
        from . import gptq as G
        import time
        t_begin = time.perf_counter()
        world, rank = self.world, self.rank
        # a linear costs its Hessian (K^2 n) plus its sequential stages (K^2 (K + N)), in comparable units
        def cost(j):
            K, N = j[0].shape
            n = sum(int(x.shape[0]) if x.dim() == 2 else int(x.numel() // x.shape[-1]) for x in j[1]) if j[1] else 0
            return float(K) * K * (0.07 * n + K + N) + 1e7        # measured: a token of the Hessian weighs ~0.07 of a (K + N) unit
        owners = assign_layers([cost(j) for j in jobs], world)
        mine = [i for i in range(len(jobs)) if owners[i] == rank]
        failure = None
        try:
            got = G.gptq_many([(jobs[i][0], jobs[i][1]) for i in mine], block_size=block_size, damping=damping, bits=bits,
                              pack=True, streams=len(self.workers))
        except (ValueError, RuntimeError) as e:      # a failure on one rank is everybody's (the others would wait forever)
            failure, got = e, []
        flag = torch.tensor([1 if failure is not None else 0], dtype=torch.int32, device='cuda')
        dist.all_reduce(flag, op=dist.ReduceOp.MAX, group=self.group_ar)
        if int(flag.item()):
            raise failure if failure is not None else ValueError('NaN when computing Hinv on another rank. Features NaN?')
        self.stats = {'reduce_bytes': 0, 'gather_bytes': 0, 'mode': 'layers'}
        results = [None] * len(jobs)
        for i, qm in zip(mine, got):
            K, N = jobs[i][0].shape
            results[i] = (qm.int_weight, qm.scale, qm.zero, (0, N))
        if gather:
            # one buffer per owner (packed bytes, scale, zero of its linears), the same layout on every rank
            sizes, place = [0] * world, {}
            for i, j in enumerate(jobs):
                K, N = j[0].shape
                o = owners[i]
                a = sizes[o]
                b4 = (a + (K // 2) * N + 255) // 256 * 256
                place[i] = (a, b4, b4 + 4 * N)
                sizes[o] = (b4 + 8 * N + 255) // 256 * 256
            flat = [torch.empty(max(sz, 1), dtype=torch.uint8, device='cuda') for sz in sizes]
            self.stats['gather_bytes'] = sum(sizes)

            def views(i):
                K, N = jobs[i][0].shape
                a, bs, bz = place[i]
                buf = flat[owners[i]]
                return (buf[a:a + (K // 2) * N].view(K // 2, N), buf[bs:bs + 4 * N].view(torch.float32),
                        buf[bz:bz + 4 * N].view(torch.float32))
            for i in mine:
                vp, vs, vz = views(i)
                vp.copy_(results[i][0])
                vs.copy_(results[i][1])
                vz.copy_(results[i][2])
            for r in range(world):
                if sizes[r] > 0:
                    dist.broadcast(flat[r], src=r, group=self.group_ag)
            for i in range(len(jobs)):
                results[i] = views(i) + ((0, jobs[i][0].shape[1]),)
        self.stats['host_issue_ms'] = 1e3 * (time.perf_counter() - t_begin)
        return results

    def run(self, jobs, n_total, block_size=128, damping=0.01, bits=4, gather=True):
        """jobs: sequence of (W (K x N, replicated), xs_local (this rank's token batches)[, ready_event]);
        `n_total` is the global token count of every job.  Returns per job (packed, scale, zero, (c0, c1)):
        the whole linear's packed weights with `gather` (column range (0, N)), else what this rank
        produced (its slab of columns, or None where it is not the owner)."""
        from . import gptq as G
        from ._lib import lib
        import time
        t_begin = time.perf_counter()
        world, rank = self.world, self.rank
        if self.mode == 'layers' and world > 1:
            return self._run_layers(list(jobs), block_size, damping, bits, gather)
        owner_mode = self.mode == 'owner' and world > 1
        main = torch.cuda.current_stream()
        start = main.record_event()
        for st in self.hstreams + [self.comm_ar, self.comm_ag] + self.workers:
            st.wait_event(start)
        jobs = list(jobs)
        if self.arenas is None:
            self.arenas = [G._Arena() for _ in self.workers]
            self.harenas = [G._Arena() for _ in self.hstreams]
        # the owner of every linear: largest sequential cost first, to the least loaded rank
        costs = [float(j[0].shape[0]) ** 2 * (j[0].shape[0] + j[0].shape[1]) + 1e7 for j in jobs]
        owners = assign_layers(costs, world)
        # issue order (the same on every rank): expensive linears first, so that their long sequential stages run
        # beside the remaining Hessians instead of after them
        order = sorted(range(len(jobs)), key=lambda i: (-costs[i], i))
        slot_free = [None] * self.nslots
        results, deferred = [None] * len(jobs), []
        self.stats = {'reduce_bytes': 0, 'gather_bytes': 0, 'mode': self.mode if world > 1 else 'single'}
        nmine = 0
        # Owner mode with `gather`: every owner collects its packed linears (bytes, then scale, then zero) in ONE
        # buffer laid out identically on all ranks and broadcasts it once, after its last linear - one collective
        # per rank instead of one per linear (the per-call host cost of a collective is what limits many ranks).
        flat, place, mine_done = None, {}, []
        if owner_mode and gather:
            sizes = [0] * world
            for i in order:
                K, N = jobs[i][0].shape
                o = owners[i]
                a = sizes[o]
                b = a + (K // 2) * N
                b4 = (b + 255) // 256 * 256
                place[i] = (a, b4, b4 + 4 * N)
                sizes[o] = (b4 + 8 * N + 255) // 256 * 256
            flat = [torch.empty(max(sz, 1), dtype=torch.uint8, device='cuda') for sz in sizes]
            self.stats['gather_bytes'] = sum(sizes)

        def views(i):
            K, N = jobs[i][0].shape
            a, bs, bz = place[i]
            buf = flat[owners[i]]
            return (buf[a:a + (K // 2) * N].view(K // 2, N), buf[bs:bs + 4 * N].view(torch.float32),
                    buf[bz:bz + 4 * N].view(torch.float32))
        for pos, i in enumerate(order):
            job = jobs[i]
            W, xs = job[0], job[1]
            x_ready = job[2] if len(job) > 2 else None       # event after which W / xs may be read (staged copies)
            K, N = W.shape
            slot = pos % self.nslots
            owner = owners[i]
            mine = (not owner_mode) or owner == rank
            hstream = self.hstreams[pos % 2]
            with torch.cuda.stream(hstream):
                if slot_free[slot] is not None:
                    hstream.wait_event(slot_free[slot])
                if x_ready is not None:
                    hstream.wait_event(x_ready)
                H = self._buf(f'H{slot}', (K, K), torch.float32, zero=True)
                hs = self._buf(f'hs{slot}', (1,), torch.int32, zero=True)
                G._ARENA = self.harenas[pos % 2]
                try:
                    G._accumulate_raw(xs, H=H, status=hs)
                finally:
                    G._ARENA = None
                if world > 1:
                    P = self._buf(f'P{slot}', (lib.jgq_hessian_lower_elems(K),), torch.float32)
                    pack_lower(H, out=P)
                ev_h = hstream.record_event()
            if world > 1:
                with torch.cuda.stream(self.comm_ar):
                    self.comm_ar.wait_event(ev_h)
                    if owner_mode:
                        dist.reduce(P, dst=owner, op=dist.ReduceOp.SUM, group=self.group_ar)
                    else:
                        dist.all_reduce(P, op=dist.ReduceOp.SUM, group=self.group_ar)
                    ev_r = self.comm_ar.record_event()
                self.stats['reduce_bytes'] += P.numel() * 4
            else:
                ev_r = ev_h
            c0, c1 = (0, N)
            if world > 1 and not owner_mode:
                c0, c1 = shard_range(N, rank, world, 16)
            packed = scale = zero = None
            if mine:
                wi = nmine % len(self.workers)
                ws = self.workers[wi]
                nmine += 1
                with torch.cuda.stream(ws):
                    ws.wait_event(ev_r)
                    if x_ready is not None:
                        ws.wait_event(x_ready)
                    if world > 1:
                        unpack_lower(P, H)
                    G._finalize_H(H, n_total)
                    slab = W[:, c0:c1].contiguous() if (c0, c1) != (0, N) else W
                    ready = ws.record_event()
                    G._ARENA = self.arenas[wi]
                    try:
                        _, _, qm = G.gptq(slab, None, block_size=block_size, damping=damping, bits=bits,
                                          return_packed=True, _defer=deferred, _hess=(H, hs, ready))
                    finally:
                        G._ARENA = None
                    packed, scale, zero = qm.int_weight, qm.scale, qm.zero
                    if flat is not None:
                        vp, vs, vz = views(i)
                        vp.copy_(packed)
                        vs.copy_(scale)
                        vz.copy_(zero)
                    slot_free[slot] = ws.record_event()
                    ev_q = slot_free[slot]
                    mine_done.append(ev_q)
            else:
                slot_free[slot] = ev_r           # the buffers of this slot are free once the reduction has read them
                ev_q = ev_r
            if flat is not None:
                results[i] = views(i) + ((0, N),)
            elif world > 1 and gather:
                with torch.cuda.stream(self.comm_ag):
                    self.comm_ag.wait_event(ev_q)
                    if x_ready is not None:
                        self.comm_ag.wait_event(x_ready)
                    widths = [shard_range(N, r, world, 16) for r in range(world)]
                    wmax = max(e - b for b, e in widths)
                    send = packed
                    if packed.shape[1] != wmax:
                        send = torch.zeros((K // 2, wmax), dtype=torch.uint8, device=packed.device)
                        send[:, :packed.shape[1]] = packed
                    recv = torch.empty((world, K // 2, wmax), dtype=torch.uint8, device=packed.device)
                    dist.all_gather_into_tensor(recv, send.contiguous(), group=self.group_ag)
                    full = torch.cat([recv[r, :, :e - b] for r, (b, e) in enumerate(widths)], dim=1)
                    for t in (packed, send, recv, full):
                        t.record_stream(self.comm_ag)
                    self.stats['gather_bytes'] += recv.numel()
                    # scale / zero depend on W alone (gptq.py:105-118): every rank computes all of them
                    Wf = W if W.dtype == torch.float32 else W.float()
                    full_params = G._col_params(Wf.contiguous())
                results[i] = (full, full_params['scale'], full_params['zero'], (0, N))
            else:
                results[i] = (packed, scale, zero, (c0, c1))
        if flat is not None:
            with torch.cuda.stream(self.comm_ag):
                for e in mine_done:
                    self.comm_ag.wait_event(e)
                for r in range(world):
                    if flat[r].numel() > 1:
                        dist.broadcast(flat[r], src=r, group=self.group_ag)
                        flat[r].record_stream(self.comm_ag)
        for st in self.hstreams + [self.comm_ar, self.comm_ag] + self.workers:
            main.wait_event(st.record_event())
        self.stats['host_issue_ms'] = 1e3 * (time.perf_counter() - t_begin)    # everything enqueued, nothing waited for yet
        st_word = 0
        if deferred:
            for w, hw in torch.stack(deferred).tolist():       # (stage status, Hessian status) per job
                st_word |= int(w) | (int(hw) << 8)
        if world > 1:            # a failure on one rank is everybody's: the status bits are OR-ed over the ranks
            bits = torch.tensor([(st_word >> k) & 1 for k in range(16)], dtype=torch.int32, device='cuda')
            dist.all_reduce(bits, op=dist.ReduceOp.MAX, group=self.group_ar)      # NCCL has no bitwise OR: MAX per bit
            st_word = sum(int(v) << k for k, v in enumerate(bits.tolist()))
        for a in self.arenas + self.harenas:
            a.release()                  # the status read above synchronised with every stream used here
        G._raise_status(st_word)
        return results
