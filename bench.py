#!/usr/bin/env python
"""Benchmark of the GPTQ hot path on B200.

Workload (one "step"): GPTQ-quantize every block linear of a GPT-2-small-shaped
model (12 blocks x {768x2304, 768x768, 768x3072, 3072x768}, fp32 weights
~0.02*N(0,1)) to 4 bits from 65536 calibration tokens (128 sequences x 512
uniform-random ids), blocksize 128, damping 0.01, then pack the result.
Calibration activations are produced once, outside the timed region, by a plain
torch forward of that architecture with each linear replaced by its quantized
weight as soon as it exists (the reference's default calibration mode).

  value : weights quantized per second, activations and weights resident in HBM
  e2e   : the same through the public host API with pinned HOST buffers: every
          step copies weights + activations host->device and the packed result
          device->host inside the timed region

`--impl reference` times the CPU oracle (NumPy/SciPy restatement of the reference,
all host cores) on a bounded sample of the same workload: one block (4 linears).
Multi-GPU (`torchrun`, one rank per GPU): ONE model, strong scaling.  The calibration
tokens of every linear are sharded over the ranks; per linear the local Hessian sums
are all-reduced over NCCL (lower triangle only, overlapped with the next Hessian
GEMM), the quantize loop is sharded over output channels, and the packed column slabs
are all-gathered.  The line also carries the layer-parallel form (one independent
model per rank, no collective) under `replicas`, and the packed matmul sharded over N.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = 'gptq_weights_quantized_per_s'
UNIT = 'weights/s'
LINEARS = (('attn.c_attn', 768, 2304), ('attn.c_proj', 768, 768), ('mlp.c_fc', 768, 3072), ('mlp.c_proj', 3072, 768))
N_LAYERS, D_MODEL, N_HEADS, VOCAB, SEQ, N_SEQ, CALIB_BATCHES = 12, 768, 12, 50257, 512, 128, 16
BLOCK_SIZE, DAMP = 128, 0.01


def workload_name(layers):
    return (f'gpt2-small-shaped GPTQ: {layers} blocks x 4 linears (768x2304, 768x768, 768x3072, 3072x768), '
            f'{N_SEQ * SEQ} calibration tokens in {CALIB_BATCHES} batches, 4-bit, blocksize {BLOCK_SIZE}, '
            f'damp {DAMP}, pack included; lm_head not quantized')


# --------------------------------------------------------------------------
# caller side: a minimal GPT-2-shaped forward that yields each linear's input
# --------------------------------------------------------------------------
def init_block(torch, gen, device):
    return {name: (0.02 * torch.randn((k, n), generator=gen, device=device, dtype=torch.float32))
            for name, k, n in LINEARS}


def block_forward(torch, h, weights, quantize_fn):
    """One transformer block.  `quantize_fn(name, W, x)` returns the weight to continue with
    (and may record x, the calibration input of that linear)."""
    F = torch.nn.functional
    B, T, D = h.shape
    x = F.layer_norm(h, (D,))
    w = quantize_fn('attn.c_attn', weights['attn.c_attn'], x)
    qkv = (x.reshape(-1, D) @ w).reshape(B, T, 3, N_HEADS, D // N_HEADS).permute(2, 0, 3, 1, 4)
    a = F.scaled_dot_product_attention(qkv[0], qkv[1], qkv[2], is_causal=True)
    a = a.transpose(1, 2).reshape(B, T, D)
    w = quantize_fn('attn.c_proj', weights['attn.c_proj'], a)
    h = h + (a.reshape(-1, D) @ w).reshape(B, T, D)
    x = F.layer_norm(h, (D,))
    w = quantize_fn('mlp.c_fc', weights['mlp.c_fc'], x)
    m = F.gelu((x.reshape(-1, D) @ w), approximate='tanh')
    w = quantize_fn('mlp.c_proj', weights['mlp.c_proj'], m.reshape(B, T, 4 * D))
    h = h + (m @ w).reshape(B, T, D)
    return h


def embed(torch, gen, device):
    ids = torch.randint(0, VOCAB, (N_SEQ, SEQ), generator=gen, device=device)
    wte = 0.02 * torch.randn((VOCAB, D_MODEL), generator=gen, device=device)
    wpe = 0.02 * torch.randn((1024, D_MODEL), generator=gen, device=device)
    return wte[ids] + wpe[:SEQ][None]


# --------------------------------------------------------------------------
# clocks
# --------------------------------------------------------------------------
class ClockSampler:
    FIELDS = ('clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,'
              'clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap')

    def __init__(self, index):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(['nvidia-smi', '-i', str(self.index), f'--query-gpu={self.FIELDS}',
                                          '--format=csv,noheader,nounits', '-lms', '100'],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {'sm_mhz': None, 'sm_max_mhz': None, 'reasons': ['nvidia-smi unavailable']}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ('hw_slowdown', 'hw_thermal_slowdown', 'sw_thermal_slowdown', 'sw_power_cap')
        for ln in self.lines:
            parts = [p.strip() for p in ln.split(',')]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0])); mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[2:6]):
                if val.lower().startswith('active'):
                    reasons.add(name)
        return {'sm_mhz': statistics.median(sm) if sm else None, 'sm_max_mhz': max(mx) if mx else None,
                'samples': len(sm), 'reasons': sorted(reasons)}


# --------------------------------------------------------------------------
# reference arm / CPU baseline: the oracle on one block
# --------------------------------------------------------------------------
def cpu_block_inputs(seed):
    """Block-0 weights and per-linear calibration inputs (fp32 forward, torch CPU ops)."""
    import torch
    gen = torch.Generator(device='cpu').manual_seed(seed)
    h = embed(torch, gen, 'cpu')
    weights = init_block(torch, gen, 'cpu')
    captured = {}

    def grab(name, W, x):
        captured[name] = x.reshape(-1, x.shape[-1]).numpy()
        return W
    block_forward(torch, h, weights, grab)
    return [(name, weights[name].numpy(), np.array_split(captured[name], CALIB_BATCHES)) for name, _, _ in LINEARS]


def cpu_block_step(items):
    from oracle import ref_gptq as R
    for _, W, xs in items:
        Q, params = R.gptq(W, xs, block_size=BLOCK_SIZE, damping=DAMP)
        R.pack_matrix(Q, params)


def cpu_threads():
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def set_blas_threads(n):
    """torchrun exports OMP_NUM_THREADS=1 to its workers; the CPU arm sets the BLAS pool itself."""
    try:
        from threadpoolctl import threadpool_limits
        threadpool_limits(limits=n)
    except Exception:
        pass
    try:
        import torch
        torch.set_num_threads(n)
    except Exception:
        pass


def blas_threads():
    try:
        from threadpoolctl import threadpool_info
        return max([int(p.get('num_threads', 1)) for p in threadpool_info() if p.get('user_api') == 'blas'] or [1])
    except Exception:
        return None


def profile_figure(fname, key):
    """A figure taken from a committed profiler summary (a line `key: value` in profiles/<fname>);
    (None, reason) when the file or the line is missing."""
    path = os.path.join(ROOT, 'profiles', fname)
    try:
        for ln in open(path):
            if ln.strip().startswith(key + ':'):
                return float(ln.split(':', 1)[1].split()[0]), f'profiles/{fname} ({key}, one ncu capture of that launch)'
    except (OSError, ValueError):
        pass
    return None, f'no {key} line in profiles/{fname}'


# --------------------------------------------------------------------------
# parity of the benchmark's own layers (checker; never inside a timed region)
# --------------------------------------------------------------------------
PARITY_MIN_SAME = 0.999      # identical-code bar
PARITY_FLOOR_FACTOR = 2.0    # ... or this many times the oracle's own fp32-rounding floor, whichever is looser
PARITY_RECON_REL = 1e-3      # relative difference of the reconstruction errors


def parity_bar(floor_mismatch):
    """Largest accepted fraction of differing codes: 1e-3, unless the oracle itself moves more codes
    than half of that when its Hessian is rounded differently (accumulated in fp64, then cast to
    fp32); then the bar is PARITY_FLOOR_FACTOR times that measured floor."""
    return max(1.0 - PARITY_MIN_SAME, PARITY_FLOOR_FACTOR * floor_mismatch)


def layer_parity(R, W, xs, codes_gpu, Q_gpu, block_size, damping, bits=4, actorder=False, cond=True):
    """Compares one GPU-quantized layer with the CPU oracle on the same bytes.  `W`, `xs`, `codes_gpu`,
    `Q_gpu` are NumPy arrays.  Returns the figures the bench line and the tests report."""
    Q_ref, p_ref, it = R.gptq(W, xs, block_size=block_size, damping=damping, bits=bits, actorder=actorder,
                              return_internals=True)
    same = float((codes_gpu == it['codes']).mean())
    e_ref = R.reconstruction_error(W, Q_ref, xs)
    e_got = R.reconstruction_error(W, Q_gpu, xs)
    # noise floor: the oracle against itself with a Hessian that differs only by fp32 rounding
    H64 = R.accumulate_H_direct(xs, use_fp64=True)
    _, _, it_f = R.gptq(W, xs, block_size=block_size, damping=damping, bits=bits, actorder=actorder,
                        H=H64.astype(np.float32), return_internals=True)
    floor_same = float((it_f['codes'] == it['codes']).mean())
    out = {'K': int(W.shape[0]), 'N': int(W.shape[1]), 'same_codes': same,
           'recon_rel': abs(e_got - e_ref) / e_ref, 'recon_err_oracle': e_ref,
           'floor_same_codes_oracle_fp64H_vs_fp32H': floor_same,
           'bar_mismatch': parity_bar(1.0 - floor_same)}
    if cond:
        ev = np.linalg.eigvalsh(H64)
        out['cond_H'] = float(ev[-1] / max(ev[0], 1e-300))
        out['cond_H_damped'] = float((ev[-1] + damping * np.mean(np.diag(H64))) /
                                     (max(ev[0], 0.0) + damping * np.mean(np.diag(H64))))
    out['ok'] = bool((1.0 - same) <= out['bar_mismatch'] and out['recon_rel'] <= PARITY_RECON_REL)
    return out


def headline_parity(torch, gg, dev, seed=2002):
    """Block 0 of the benchmark workload (same generator, same forward as the timed run): every linear is
    quantized on the GPU from the activations the forward produces with the previous quantized weights in
    place, and the CPU oracle quantizes the same weight from the same activation bytes."""
    from oracle import ref_gptq as R
    gen = torch.Generator(device=dev).manual_seed(seed)
    h = embed(torch, gen, dev)
    weights = init_block(torch, gen, dev)
    rows = {}

    def quantize_and_check(name, W, x):
        xs = x.reshape(-1, x.shape[-1]).contiguous()
        chunks = list(xs.chunk(CALIB_BATCHES))
        Q, _, codes = gg.gptq(W, chunks, block_size=BLOCK_SIZE, damping=DAMP, return_codes=True)
        rows[name] = layer_parity(R, W.cpu().numpy(), [c.cpu().numpy() for c in chunks], codes.cpu().numpy(),
                                  Q.cpu().numpy(), BLOCK_SIZE, DAMP)
        return Q
    block_forward(torch, h, weights, quantize_and_check)
    return rows


def run_reference(args):
    rank = int(os.environ.get('RANK', '0'))
    if rank != 0:
        return
    threads = cpu_threads()
    set_blas_threads(threads)
    items = cpu_block_inputs(2002)
    weights = sum(W.size for _, W, _ in items)
    for _ in range(args.warmup):
        cpu_block_step(items)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_block_step(items)
    dt = (time.perf_counter() - t0) / args.steps
    val = weights / dt
    sample = 'one block (4 linears, 7.08 M weights) of the workload per step, 65536 calibration tokens'
    line = {'impl': 'reference', 'metric': METRIC, 'value': val, 'unit': UNIT, 'n_gpus': args.gpus,
            'steps': args.steps, 'warmup': args.warmup, 'ms_per_step': dt * 1e3, 'higher_is_better': True,
            'scaling': 'weak', 'vs_baseline': None, 'dtype': 'f32', 'data': 'synthetic',
            'config': {'workload': workload_name(N_LAYERS), 'sample': sample},
            'cpu_baseline': {'value': val, 'unit': UNIT, 'cores': threads, 'blas_threads': blas_threads(),
                             'kind': 'port', 'sample': sample},
            'e2e': {'value': val, 'unit': UNIT, 'h2d_bytes_per_step': 0, 'd2h_bytes_per_step': 0}}
    print(json.dumps(line), flush=True)



def e2e_single(torch, gg, args, dev, model, acts, layers, total_weights, barrier):
    """End to end on one GPU: weights and calibration inputs in pinned host memory, every step copies them to
    the device (overlapped with compute by gptq_many) and the packed result back."""
    world = 1
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    free_host = 0
    try:
        for ln in open('/proc/meminfo'):
            if ln.startswith('MemAvailable'):
                free_host = int(ln.split()[1]) * 1024
    except OSError:
        pass
    per_layer = sum(a.numel() * 4 for a in acts[0].values())
    budget = min(free_host // (2 * max(world, 1)), 24 << 30) if free_host else 4 << 30
    distinct = max(1, min(layers, budget // per_layer))
    host_acts = [{k: v.cpu().pin_memory() for k, v in acts[i].items()} for i in range(distinct)]
    host_w = [{k: v.cpu().pin_memory() for k, v in m.items()} for m in model]
    host_out = [{name: (torch.empty((k // 2, n), dtype=torch.uint8).pin_memory(),
                        torch.empty(n, dtype=torch.float32).pin_memory(),
                        torch.empty(n, dtype=torch.float32).pin_memory()) for name, k, n in LINEARS}
                for _ in range(layers)]
    acts_dev_bytes = sum(v.numel() * 4 for a in acts for v in a.values())
    torch.cuda.empty_cache()
    h2d = sum(host_acts[i % distinct][name].numel() * 4 + host_w[i][name].numel() * 4
              for i in range(layers) for name, _, _ in LINEARS)
    d2h = sum(sum(t.numel() * t.element_size() for t in host_out[i][name])
              for i in range(layers) for name, _, _ in LINEARS)

    def step_e2e():
        jobs = [(host_w[i][name], list(host_acts[i % distinct][name].chunk(CALIB_BATCHES)))
                for i in range(layers) for name, _, _ in LINEARS]
        outs = [host_out[i][name] for i in range(layers) for name, _, _ in LINEARS]
        gg.gptq_many(jobs, block_size=BLOCK_SIZE, damping=DAMP, pack=True, out_host=outs, streams=args.streams,
                     hessian_stream=not args.no_hessian_stream)
        torch.cuda.synchronize()

    for _ in range(min(args.warmup, 3)):
        step_e2e()
    barrier()
    e0.record()
    for _ in range(args.steps):
        step_e2e()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / args.steps], device=dev, dtype=torch.float64)
    e2e_ms = float(t.item())
    e2e = {'value': world * total_weights / (e2e_ms * 1e-3), 'unit': UNIT, 'ms_per_step': e2e_ms,
           'h2d_bytes_per_step': h2d, 'd2h_bytes_per_step': d2h,
           'distinct_activation_sets_in_pinned_memory': distinct}
    del host_acts, host_w, host_out
    return e2e, acts_dev_bytes


def e2e_sharded(torch, dist, args, dev, rank, world, model, acts, pipe, shard, total_weights, barrier):
    """End to end on N GPUs: every rank holds ITS token shard of every calibration input and the weights in
    pinned host memory; a step copies them to the device (copy stream, one event per linear), runs the
    sharded pipeline on them and rank 0 reads the packed model back."""
    b, e = shard
    layers = len(model)
    host_acts = [{k: v[b:e].cpu().pin_memory() for k, v in a.items()} for a in acts]
    host_w = [{k: v.cpu().pin_memory() for k, v in m.items()} for m in model]
    dev_acts = [{k: torch.empty_like(v, device=dev) for k, v in a.items()} for a in host_acts]
    dev_w = [{k: torch.empty_like(v, device=dev) for k, v in m.items()} for m in host_w]
    host_out = [{name: torch.empty((k // 2, n), dtype=torch.uint8).pin_memory() for name, k, n in LINEARS} for _ in range(layers)]
    copier = torch.cuda.Stream()
    h2d = sum(v.numel() * 4 for a in host_acts for v in a.values()) + sum(v.numel() * 4 for m in host_w for v in m.values())
    d2h = sum(t.numel() for o in host_out for t in o.values())
    nb = max(1, CALIB_BATCHES // world)

    def step():
        jobs = []
        copier.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(copier):
            for i in range(layers):
                for name, _, _ in LINEARS:
                    dev_w[i][name].copy_(host_w[i][name], non_blocking=True)
                    dev_acts[i][name].copy_(host_acts[i][name], non_blocking=True)
                    jobs.append((dev_w[i][name], list(dev_acts[i][name].chunk(nb)), copier.record_event()))
        res = pipe.run(jobs, N_SEQ * SEQ, block_size=BLOCK_SIZE, damping=DAMP)
        if rank == 0:
            j = 0
            for i in range(layers):
                for name, _, _ in LINEARS:
                    host_out[i][name].copy_(res[j][0], non_blocking=True)
                    j += 1
        torch.cuda.synchronize()

    for _ in range(min(args.warmup, 3)):
        step()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / args.steps], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    return {'value': total_weights / (ms * 1e-3), 'unit': UNIT, 'ms_per_step': ms,
            'h2d_bytes_per_step': h2d * world, 'd2h_bytes_per_step': d2h,
            'h2d_bytes_per_step_per_rank': h2d, 'h2d_GBps_per_rank': h2d / (ms * 1e-3) / 1e9,
            'what': 'one model on all ranks: each rank copies its token shard of every calibration input and the weights '
                    'host->device, rank 0 reads the packed model back'}

# --------------------------------------------------------------------------
# our arm
# --------------------------------------------------------------------------
def run_ours(args):
    import torch
    import torch.distributed as dist
    import jax_gptq_b200 as G
    import importlib
    gg = importlib.import_module('jax_gptq_b200.gptq')
    from jax_gptq_b200._lib import lib

    world = int(os.environ.get('WORLD_SIZE', '1'))
    rank = int(os.environ.get('RANK', '0'))
    local = int(os.environ.get('LOCAL_RANK', '0'))
    torch.cuda.set_device(local)
    dev = torch.device('cuda', local)
    if world > 1:
        dist.init_process_group('nccl', device_id=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    layers = args.layers
    gen = torch.Generator(device=dev).manual_seed(2002)       # the same model on every rank

    # ---- untimed set-up: weights, and calibration inputs captured with quantized weights in place ----
    h = embed(torch, gen, dev)
    model, acts = [], []
    t_fwd0 = time.perf_counter()
    for _ in range(layers):
        weights = init_block(torch, gen, dev)
        captured = {}

        def quantize_in_place(name, W, x):
            xs = x.reshape(-1, x.shape[-1]).contiguous()
            captured[name] = xs
            Q, _ = gg.gptq(W, list(xs.chunk(CALIB_BATCHES)), block_size=BLOCK_SIZE, damping=DAMP)
            return Q
        h = block_forward(torch, h, weights, quantize_in_place)
        model.append(weights)
        acts.append(captured)
    torch.cuda.synchronize()
    setup_s = time.perf_counter() - t_fwd0
    del h
    total_weights = layers * sum(k * n for _, k, n in LINEARS)

    def step_resident():
        jobs = [(weights[name], list(captured[name].chunk(CALIB_BATCHES)))
                for weights, captured in zip(model, acts) for name, _, _ in LINEARS]
        return gg.gptq_many(jobs, block_size=BLOCK_SIZE, damping=DAMP, pack=True, streams=args.streams, hessian_stream=not args.no_hessian_stream)

    # ---- value: device-resident ----
    for _ in range(args.warmup):
        step_resident()
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    launches0 = lib.jgq_launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step_resident()
    e1.record()
    torch.cuda.synchronize()
    launches = lib.jgq_launch_count() - launches0
    ms = e0.elapsed_time(e1) / args.steps
    clocks = sampler.stop() if rank == 0 else None
    t = torch.tensor([ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_max = float(t.item())
    value = world * total_weights / (ms_max * 1e-3)

    # ---- N > 1: one model, tokens sharded over the ranks (strong scaling) ----
    replicas = None
    sharded = None
    layer_parallel = None
    headline_split = None
    if world > 1:
        from jax_gptq_b200 import dist as D
        replicas = {'value': value, 'unit': UNIT, 'ms_per_step': ms_max, 'scaling': 'weak',
                    'what': f'{world} independent models, one per GPU, no data-path collective'}
        n_tok = N_SEQ * SEQ
        b, e = D.shard_range(n_tok, rank, world, 64)
        pipe = D.ShardedPipeline(streams=min(args.streams, 8))

        def sharded_jobs():
            return [(weights[name], list(captured[name][b:e].chunk(max(1, CALIB_BATCHES // world))))
                    for weights, captured in zip(model, acts) for name, _, _ in LINEARS]

        def step_sharded():
            return pipe.run(sharded_jobs(), n_tok, block_size=BLOCK_SIZE, damping=DAMP)
        for _ in range(args.warmup):
            out_sh = step_sharded()
        barrier()
        launches0 = lib.jgq_launch_count()
        e0.record()
        for _ in range(args.steps):
            out_sh = step_sharded()
        e1.record()
        torch.cuda.synchronize()
        launches = lib.jgq_launch_count() - launches0
        t = torch.tensor([e0.elapsed_time(e1) / args.steps], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_max = float(t.item())
        value = total_weights / (ms_max * 1e-3)           # ONE model: strong scaling
        # collective alone: the all-reduces of one step, back to back
        bufs = [torch.zeros(lib.jgq_hessian_lower_elems(k), dtype=torch.float32, device=dev) for _, k, _ in LINEARS]
        for _ in range(2):
            for j, bf in enumerate(bufs):
                dist.reduce(bf, dst=j % world)
        barrier()
        e0.record()
        for li in range(layers):
            for j, bf in enumerate(bufs):
                dist.reduce(bf, dst=(li + j) % world)
        e1.record()
        torch.cuda.synchronize()
        ar_ms = e0.elapsed_time(e1)
        # check: the sharded result of block 0 against the single-GPU path on the same data
        same = []
        for j, (name, _, _) in enumerate(LINEARS):
            Q1, p1 = gg.gptq(model[0][name], list(acts[0][name].chunk(CALIB_BATCHES)), block_size=BLOCK_SIZE, damping=DAMP)
            ref_packed = G.pack_matrix(Q1, p1).int_weight
            got = out_sh[j][0]
            lo = ((got & 15) == (ref_packed & 15)).float().mean()
            hi = ((got >> 4) == (ref_packed >> 4)).float().mean()
            same.append(float((lo + hi) / 2))
        sharded = {'collective': 'NCCL reduce (sum, fp32) of the lower block triangle of every Hessian to the linear\'s owner rank, '
                                 'one per linear; one broadcast per owner rank of its packed linears (bytes, scale, zero) on a second communicator',
                   'mode': pipe.stats.get('mode'),
                   'reduce_bytes_per_step': pipe.stats['reduce_bytes'], 'broadcast_bytes_per_step': pipe.stats['gather_bytes'],
                   'reduce_ms_alone_per_step': ar_ms, 'reduce_share_of_step': ar_ms / ms_max,
                   'host_issue_ms_rank0_last_step': pipe.stats.get('host_issue_ms'),
                   'tokens_per_rank': e - b,
                   'check_same_codes_block0_vs_single_gpu': same,
                   'check_note': 'the sharded Hessian differs from the single-GPU one by fp32 summation order only; on the K = 3072 '
                                 'layer that moves about as many codes as the oracle\'s own rounding floor (see parity)',
                   'check_ok': bool(min(same) >= 0.998)}

        # ---- the other split of one model: linears (not tokens) sharded over the ranks, no Hessian travels ----
        pipe_l = D.ShardedPipeline(streams=args.streams, mode='layers')

        def full_jobs():
            return [(weights[name], list(captured[name].chunk(CALIB_BATCHES)))
                    for weights, captured in zip(model, acts) for name, _, _ in LINEARS]

        def step_layers():
            return pipe_l.run(full_jobs(), n_tok, block_size=BLOCK_SIZE, damping=DAMP)
        for _ in range(args.warmup):
            out_l = step_layers()
        barrier()
        launches0 = lib.jgq_launch_count()
        e0.record()
        for _ in range(args.steps):
            out_l = step_layers()
        e1.record()
        torch.cuda.synchronize()
        launches_l = lib.jgq_launch_count() - launches0
        t = torch.tensor([e0.elapsed_time(e1) / args.steps], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_layers = float(t.item())
        same_l = []
        for j, (name, _, _) in enumerate(LINEARS):          # same tokens, same kernels: the bytes must be the single-GPU ones
            Q1, p1 = gg.gptq(model[0][name], list(acts[0][name].chunk(CALIB_BATCHES)), block_size=BLOCK_SIZE, damping=DAMP)
            same_l.append(bool(torch.equal(out_l[j][0], G.pack_matrix(Q1, p1).int_weight)))
        layer_parallel = {'value': total_weights / (ms_layers * 1e-3), 'unit': UNIT, 'ms_per_step': ms_layers, 'scaling': 'strong',
                          'what': f'one model on {world} GPUs, every linear quantized entirely by its owner rank from all of its '
                                  'tokens (activations resident on every rank); the only collectives are the owners\' result '
                                  'broadcasts', 'broadcast_bytes_per_step': pipe_l.stats['gather_bytes'],
                          'host_issue_ms_rank0_last_step': pipe_l.stats.get('host_issue_ms'),
                          'check_block0_bit_identical_to_single_gpu': same_l, 'check_ok': all(same_l)}
        sharded['value'] = value
        sharded['ms_per_step'] = ms_max
        headline_split = 'tokens'
        if ms_layers < ms_max and all(same_l):
            # the headline is the faster split of the SAME job (one model, N GPUs); the token split stays under `sharded`
            value, ms_max, launches, headline_split = layer_parallel['value'], ms_layers, launches_l, 'layers'

    # ---- the same work issued one linear at a time, in the order the calibration forward needs the
    # quantized weights (layer l+1's input depends on layer l's result): nothing overlaps ----
    def step_in_order():
        for weights, captured in zip(model, acts):
            for name, _, _ in LINEARS:
                gg.gptq_many([(weights[name], list(captured[name].chunk(CALIB_BATCHES)))], block_size=BLOCK_SIZE,
                             damping=DAMP, pack=True, streams=1, hessian_stream=not args.no_hessian_stream)
    step_in_order()
    torch.cuda.synchronize()
    e0.record()
    step_in_order()
    e1.record()
    torch.cuda.synchronize()
    ms_in_order = e0.elapsed_time(e1)

    # ---- roofline of the dominant kernel: Hessian accumulation of the K=3072 linear ----
    x_big = acts[0]['mlp.c_proj']
    n_tok, Kb = x_big.shape
    batches = list(x_big.chunk(CALIB_BATCHES))
    for _ in range(2):
        gg._accumulate_raw(batches)
    torch.cuda.synchronize()
    reps = 5
    l0 = lib.jgq_launch_count()
    e0.record()
    for _ in range(reps):
        gg._accumulate_raw(batches)
    e1.record()
    torch.cuda.synchronize()
    h_launches = (lib.jgq_launch_count() - l0) / reps
    h_ms = e0.elapsed_time(e1) / reps
    flops = 2.0 * n_tok * Kb * Kb
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, 'MEASURED_PEAKS.json')))
    except (OSError, ValueError):
        pass
    # the stage is timed alone, a few milliseconds at a time: the burst peak is the denominator
    peak_tf = float(peaks.get('bf16_tflops', 1590.0))
    peak_sus = float(peaks.get('bf16_tflops_sustained', 1400.0))
    achieved_tf = flops / (h_ms * 1e-3) / 1e12
    traffic, traffic_src = profile_figure('hessian_pair_k3072_gpt2_block.md', 'dram_bytes_per_launch')
    roofline = {'kernel': 'hessian_accum (H += X^T X, K=3072, n=65536, 16 batches)', 'bound': 'tensor',
                'achieved': achieved_tf, 'peak': peak_tf, 'unit': 'TFLOP/s', 'frac': achieved_tf / peak_tf,
                'peak_source': ('MEASURED_PEAKS.json bf16_tflops (burst: the stage is timed in isolation)' if peaks
                                else 'fallback 1.59 PFLOP/s burst'),
                'frac_of_sustained_peak': achieved_tf / peak_sus,
                'launches_per_hessian': h_launches, 'ms_per_hessian': h_ms,
                'note': 'time covers every launch of one Hessian (operand split, tcgen05 kernel, slice reduction)',
                'traffic': traffic, 'traffic_source': traffic_src}

    # ---- per-stage device time of one block (explains `value`; not part of it) ----
    stages = {}

    def timed(label, fn):
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        r = fn()
        b.record()
        torch.cuda.synchronize()
        stages[label] = stages.get(label, 0.0) + a.elapsed_time(b)
        return r
    for rep in range(2):              # first pass warms up, second is recorded
        stages.clear()
        for name, k, n in LINEARS:
            xs_l = list(acts[0][name].chunk(CALIB_BATCHES))
            Wf = model[0][name].clone()
            tag = f'K{k}xN{n}'
            p = timed(f'{tag}.col_params', lambda: gg._col_params(Wf))
            Hn = timed(f'{tag}.hessian', lambda: gg._accumulate_raw(xs_l))
            Hf = timed(f'{tag}.finalize', lambda: gg._finalize_H(*Hn))
            Ls = timed(f'{tag}.damp_invert', lambda: gg._damp_and_invert(Wf, Hf, DAMP))
            Qc = timed(f'{tag}.quantize', lambda: gg._quantize(Wf, Ls[0], p, BLOCK_SIZE, torch.float32))
            timed(f'{tag}.pack', lambda: G.pack_matrix(Qc[0], p))
    stages = {k2: round(v, 4) for k2, v in stages.items()}

    # ---- e2e: pinned host buffers in, packed result out, all copies inside the timed region ----
    if world > 1:
        e2e = e2e_sharded(torch, dist, args, dev, rank, world, model, acts, pipe, (b, e), total_weights, barrier)
        acts_dev_bytes = sum(v.numel() * 4 for a in acts for v in a.values())
        del acts, model, x_big, batches
        torch.cuda.empty_cache()
    else:
        model_h, acts_h = model, acts
        del acts, model, x_big, batches
        e2e, acts_dev_bytes = e2e_single(torch, gg, args, dev, model_h, acts_h, layers, total_weights, barrier)
        del model_h, acts_h

    # ---- packed-int4 matmul: HBM GB/s at M=1, TFLOP/s at M=2048 (single rank numbers) ----
    w4 = []
    if rank == 0 and not args.skip_matmul:
        w4 = bench_w4(torch, G, dev, peaks)

    w4_sharded = None
    if world > 1 and not args.skip_matmul:
        w4_sharded = bench_w4_sharded(torch, dist, dev, rank, world, peaks)

    cpu_baseline = None
    if rank == 0 and world == 1 and not args.skip_cpu:
        set_blas_threads(cpu_threads())
        items = cpu_block_inputs(2002)
        cpu_block_step(items)                 # warm-up pass (BLAS thread pool, page faults)
        t0 = time.perf_counter()
        for _ in range(2):
            cpu_block_step(items)
        dt = (time.perf_counter() - t0) / 2
        cpu_baseline = {'value': sum(W.size for _, W, _ in items) / dt, 'unit': UNIT, 'cores': cpu_threads(),
                        'blas_threads': blas_threads(), 'kind': 'port', 'seconds_per_pass': dt,
                        'sample': 'one block (4 linears, 7.08 M weights), 65536 calibration tokens, NumPy/SciPy oracle, '
                                  'one warm-up pass then the mean of two'}

    parity = None
    if rank == 0 and not args.skip_cpu and not args.skip_parity:
        parity = headline_parity(torch, gg, dev, seed=2002)

    if rank == 0:
        line = {'metric': METRIC, 'value': value, 'unit': UNIT, 'n_gpus': world, 'steps': args.steps,
                'warmup': args.warmup, 'ms_per_step': ms_max, 'higher_is_better': True,
                'scaling': 'strong' if world > 1 else 'weak',
                'vs_baseline': None, 'dtype': 'f32', 'data': 'synthetic',
                'config': {'workload': workload_name(layers), 'weights_per_step': total_weights,
                           'l2': 'inputs larger than L2 (each linear reads 0.2-0.8 GB of activations)',
                           'parallelism': ((f'one model on {world} GPUs, both splits measured, headline = the faster one: '
                                            + ('linears sharded over the ranks (each quantized by its owner from all tokens), results broadcast'
                                               if headline_split == 'layers' else
                                               'calibration tokens sharded, Hessians reduced to an owner rank per linear (NCCL), results broadcast'))
                                           if world > 1 else 'one GPU'),
                           'linears_in_flight_per_gpu': args.streams,
                           'resident_activation_bytes_per_gpu': acts_dev_bytes, 'setup_seconds': setup_s},
                'clocks': clocks, 'e2e': e2e, 'gpu_launches': int(launches), 'roofline': roofline,
                'cpu_baseline': cpu_baseline, 'stage_ms_one_block': stages, 'w4_matmul': w4,
                'ms_per_step_one_linear_at_a_time': ms_in_order,
                'value_note': 'the 48 linears are issued as independent jobs (calibration inputs captured beforehand); '
                              'ms_per_step_one_linear_at_a_time is the same work with nothing overlapped, the order a '
                              'calibration forward with quantized weights in place imposes',
                'parity': parity, 'replicas': replicas, 'sharded': sharded, 'layer_parallel': layer_parallel,
                'w4_matmul_sharded': w4_sharded}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()



# --------------------------------------------------------------------------
# sized workloads: Llama-7B-shaped linears and one 70B-shaped block (bf16 weights and activations)
# --------------------------------------------------------------------------
SIZED = {
    # name: (distinct linears (K, N, how many per block), calibration tokens, bits to run, blocks in the model)
    'llama7b-linear': (((4096, 4096, 4), (4096, 11008, 2), (11008, 4096, 1)), 128 * 2048, (4,), 32),
    'llama70b-block': (((8192, 8192, 2), (8192, 1024, 2), (8192, 28672, 2), (28672, 8192, 1)), 65536, (4, 3), 1),
}
ORACLE_MAX_K = 8192          # the CPU oracle is run up to this contraction size ...
ORACLE_COLS = 512            # ... on this many output channels (channels are independent given the factor)


def run_sized(args):
    """One linear per distinct shape of the workload: bf16 W ~ 0.02 N(0,1), bf16 X ~ N(0,1) (the configuration's
    calibration data is random by definition), GPTQ + pack, per-stage device time.  Checks: up to K = 8192 the
    CPU oracle on a slice of the output channels (identical codes, reconstruction error); above that the
    residual of the factor, the status word, and the reconstruction error against round-to-nearest."""
    import importlib
    import torch
    import torch.distributed as dist
    import jax_gptq_b200 as G
    gg = importlib.import_module('jax_gptq_b200.gptq')
    from jax_gptq_b200._lib import lib
    world = int(os.environ.get('WORLD_SIZE', '1'))
    rank = int(os.environ.get('RANK', '0'))
    local = int(os.environ.get('LOCAL_RANK', '0'))
    torch.cuda.set_device(local)
    dev = torch.device('cuda', local)
    pipe = None
    if world > 1:
        dist.init_process_group('nccl', device_id=dev)
        from jax_gptq_b200 import dist as D
        pipe = D.ShardedPipeline(streams=2)
    shapes, n_tok, bit_list, blocks = SIZED[args.workload]
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, 'MEASURED_PEAKS.json')))
    except (OSError, ValueError):
        pass
    seed = 4004 if args.workload.startswith('llama7b') else 5005
    rows, total_ms, total_weights = [], 0.0, 0
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    for (K, N, count) in shapes:
        gen = torch.Generator(device=dev).manual_seed(seed + K + N)
        W = (0.02 * torch.randn((K, N), generator=gen, device=dev)).bfloat16()
        X = torch.empty((n_tok, K), dtype=torch.bfloat16, device=dev)
        for r0 in range(0, n_tok, 16384):                   # generated in pieces: no fp32 copy of the whole batch
            X[r0:r0 + 16384] = torch.randn((min(16384, n_tok - r0), K), generator=gen, device=dev).bfloat16()
        b, e = (0, n_tok)
        if world > 1:
            b, e = D.shard_range(n_tok, rank, world, 64)
        xs = list(X[b:e].chunk(max(1, 16 // world)))
        for bits in bit_list:
            def one():
                if world > 1:
                    return pipe.run([(W, xs)], n_tok, block_size=BLOCK_SIZE, damping=DAMP, bits=bits)[0]
                Q, params = gg.gptq(W, xs, block_size=BLOCK_SIZE, damping=DAMP, bits=bits)
                return G.pack_matrix(Q, params)
            for _ in range(max(1, min(args.warmup, 2))):
                one()
            torch.cuda.synchronize()
            if world > 1:
                dist.barrier()
            reps = max(1, min(args.steps, 3))
            e0.record()
            for _ in range(reps):
                one()
            e1.record()
            torch.cuda.synchronize()
            t = torch.tensor([e0.elapsed_time(e1) / reps], device=dev, dtype=torch.float64)
            if world > 1:
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
            row = {'K': K, 'N': N, 'bits': bits, 'per_block': count, 'ms': ms, 'weights_per_s': K * N / (ms * 1e-3)}
            if rank == 0 and world == 1:
                row.update(sized_stages(torch, gg, G, W, xs, bits))
                if not args.skip_parity:
                    # the CPU oracle runs for the first bit width of every shape and for the second one on the
                    # smallest shape only (it takes about a minute per run at these sizes)
                    with_oracle = bits == bit_list[0] or N <= 1024
                    row['check'] = sized_check(torch, gg, W, xs, bits, K, N, with_oracle)
            rows.append(row)
            if bits == bit_list[0]:
                total_ms += ms * count
                total_weights += K * N * count
        del W, X, xs
        torch.cuda.empty_cache()
    clocks = sampler.stop() if rank == 0 else None
    if rank == 0:
        big = max((r for r in rows if 'stage_ms' in r), key=lambda r: r['stage_ms']['hessian'], default=None)
        roofline = None
        if big is not None:
            flops = 2.0 * n_tok * big['K'] * big['K']
            peak = float(peaks.get('bf16_tflops', 1590.0))
            ach = flops / (big['stage_ms']['hessian'] * 1e-3) / 1e12
            roofline = {'kernel': f"hessian_accum (H += X^T X, K={big['K']}, n={n_tok}, bf16 activations)", 'bound': 'tensor',
                        'achieved': ach, 'peak': peak, 'unit': 'TFLOP/s', 'frac': ach / peak,
                        'peak_source': 'MEASURED_PEAKS.json bf16_tflops (burst: the stage is timed in isolation)' if peaks else 'fallback',
                        'traffic': None}
        line = {'metric': METRIC, 'value': total_weights / (total_ms * 1e-3), 'unit': UNIT, 'n_gpus': world,
                'steps': max(1, min(args.steps, 3)), 'warmup': max(1, min(args.warmup, 2)), 'ms_per_step': total_ms,
                'higher_is_better': True, 'scaling': 'strong' if world > 1 else 'weak', 'vs_baseline': None,
                'dtype': 'f32 (bf16 weights and activations in, fp32 arithmetic)', 'data': 'synthetic',
                'config': {'workload': f'{args.workload}: one linear per distinct shape, weighted by its count per block '
                                       f'({blocks} block(s) in the model), {n_tok} calibration tokens, blocksize {BLOCK_SIZE}, damp {DAMP}',
                           'l2': 'inputs larger than L2'},
                'clocks': clocks, 'layers': rows, 'roofline': roofline,
                'model_seconds_extrapolated': total_ms * 1e-3 * blocks,
                'note': 'ms_per_step = one block (each distinct linear timed alone, times its count); the whole-model '
                        'figure multiplies by the number of blocks (extrapolated, identical shapes)'}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def sized_stages(torch, gg, G, W, xs, bits):
    stages = {}

    def timed(label, fn):
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        r = fn()
        b.record()
        torch.cuda.synchronize()
        stages[label] = round(a.elapsed_time(b), 4)
        return r
    Wf = W.float()
    p = timed('col_params', lambda: gg._col_params(Wf, bits))
    Hn = timed('hessian', lambda: gg._accumulate_raw(xs))
    Hf = timed('finalize', lambda: gg._finalize_H(*Hn))
    Ls = timed('damp_invert', lambda: gg._damp_and_invert(Wf, Hf, DAMP))
    Qc = timed('quantize', lambda: gg._quantize(Wf, Ls[0], p, BLOCK_SIZE, torch.bfloat16))
    timed('pack', lambda: G.pack_matrix(Qc[0], p))
    return {'stage_ms': stages, 'status': int(Ls[1].item())}


def sized_check(torch, gg, W, xs, bits, K, N, with_oracle=True):
    """Parity of one sized linear (see run_sized)."""
    out = {}
    n = sum(x.shape[0] for x in xs)
    H, _ = gg._accumulate_raw(xs)
    H = gg._finalize_H(H, n)
    Hd = H.double()
    Q, params, codes = gg.gptq(W, xs, block_size=BLOCK_SIZE, damping=DAMP, bits=bits, return_codes=True)
    Wd, Qd = W.double(), Q.double()
    D = Wd - Qd
    err_gptq = float((D * (Hd @ D)).sum())
    # round to nearest with the same grid
    sc, z, maxq = params['scale'].double(), params['zero'].double(), params['maxq']
    Qr = sc * (torch.clamp(torch.round(Wd / sc) + z, 0, maxq) - z)
    Dr = Wd - Qr
    out['recon_err_gptq_over_rtn'] = err_gptq / float((Dr * (Hd @ Dr)).sum())
    # residual of the factor: L L^T (H + damp) = I
    Wf = W.float()
    L, status = gg._damp_and_invert(Wf, H.clone(), DAMP)
    out['status'] = int(status.item())
    Ld = L.double()
    Hdamp = Hd + torch.eye(K, device=H.device, dtype=torch.float64) * (float(torch.diagonal(H).mean()) * DAMP)
    R1 = Ld.T @ Hdamp
    resid = Ld @ R1 - torch.eye(K, device=H.device, dtype=torch.float64)
    out['factor_residual_max'] = float(resid.abs().max())
    del R1, resid, Ld, Hdamp
    if K <= ORACLE_MAX_K and with_oracle:
        from oracle import ref_gptq as R
        cols = min(N, ORACLE_COLS)
        Wn = W[:, :cols].float().cpu().numpy()
        xs_np = [x.float().cpu().numpy() for x in xs]
        Q_ref, p_ref, it = R.gptq(Wn, xs_np, block_size=BLOCK_SIZE, damping=DAMP, bits=bits, return_internals=True)
        # the GPU result for the same channels (channels are independent given the factor; scale / zero are per channel)
        same = float((codes[:, :cols].cpu().numpy() == it['codes']).mean())
        H64 = R.accumulate_H_direct(xs_np, use_fp64=True)
        _, _, it_f = R.gptq(Wn, xs_np, block_size=BLOCK_SIZE, damping=DAMP, bits=bits, H=H64.astype(np.float32), return_internals=True)
        floor_same = float((it_f['codes'] == it['codes']).mean())
        e_ref = R.reconstruction_error(Wn, Q_ref, xs_np)
        e_got = R.reconstruction_error(Wn, Q[:, :cols].float().cpu().numpy(), xs_np)
        out.update({'oracle_channels': cols, 'same_codes': same, 'floor_same_codes_oracle_fp64H_vs_fp32H': floor_same,
                    'bar_mismatch': parity_bar(1.0 - floor_same), 'recon_rel': abs(e_got - e_ref) / e_ref,
                    'ok': bool(1.0 - same <= parity_bar(1.0 - floor_same) and abs(e_got - e_ref) / e_ref <= PARITY_RECON_REL)})
    return out


def bench_w4(torch, G, dev, peaks, cases=None, no_settled=False):
    """Config-3 sweep on one GPU: fp16 activations, fp16 scale/zero; weights rotated over
    enough distinct buffers to exceed L2 between launches."""
    hbm = float(peaks.get('hbm_gbs', 6650.0))
    tf = float(peaks.get('bf16_tflops_sustained', 1400.0))
    rows = []
    gen = torch.Generator(device=dev).manual_seed(3003)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    shapes = ((4096, 4096), (4096, 11008), (11008, 4096), (8192, 28672))
    ref_us = {}       # the reference's Triton kernel on a B200, recorded by tests/golden/make_kernel_golden.py
    try:
        for r in json.load(open(os.path.join(ROOT, 'tests', 'golden', 'triton_ref_times.json')))['rows']:
            ref_us[(r['K'], r['N'], r['M'])] = r['triton_ref_us']
    except (OSError, ValueError, KeyError):
        pass
    from jax_gptq_b200 import _lib
    if cases:
        shapes = tuple(dict.fromkeys((k, n) for k, n, _ in cases))
    for K, N in shapes:
        wbytes = K * N // 2
        nbuf = max(2, -(-(300 << 20) // wbytes))
        packed = [torch.randint(0, 256, (K // 2, N), generator=gen, device=dev, dtype=torch.uint8) for _ in range(nbuf)]
        scale = (0.001 + 0.019 * torch.rand(N, generator=gen, device=dev)).half()
        zero = torch.randint(0, 16, (N,), generator=gen, device=dev).half()
        qms = [G.QuantizedMatrix(p, zero, scale) for p in packed]
        for M in ((1, 16, 128, 2048) if not cases else tuple(m for k, n, m in cases if (k, n) == (K, N))):
            x = torch.randn((M, K), generator=gen, device=dev).half()
            iters = 20 if M <= 128 else 3
            # launched straight through the C ABI so that host-side Python time does not
            # leave the GPU idle between these microsecond-scale kernels
            from jax_gptq_b200 import _lib
            need = _lib.lib.jgq_w4_matmul_workspace_bytes(M, N, K, 0)
            ws = torch.zeros(max(need, 1), dtype=torch.uint8, device=dev)
            out = torch.empty((M, N), dtype=torch.float16, device=dev)
            def launch(i, st):
                # the weights were generated long before these launches: JGQ_W4_WEIGHTS_SETTLED holds
                _lib.check(_lib.lib.jgq_w4_matmul(x.data_ptr(), _lib.F16, packed[i % nbuf].data_ptr(), zero.data_ptr(),
                                                  scale.data_ptr(), _lib.F16, out.data_ptr(), M, N, K,
                                                  0 if no_settled else _lib.W4_WEIGHTS_SETTLED,
                                                  ws.data_ptr(), need, st))
            st = torch.cuda.current_stream().cuda_stream
            for i in range(3):
                launch(i, st)
            torch.cuda.synchronize()
            e0.record()
            for i in range(iters):
                launch(i, st)
            e1.record()
            torch.cuda.synchronize()
            ms_loop = e0.elapsed_time(e1) / iters
            # the same launches recorded once into a CUDA graph and replayed: at a few microseconds per
            # kernel the Python call per launch would otherwise leave the GPU idle between kernels
            ms = ms_loop
            try:
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph):
                    cst = torch.cuda.current_stream().cuda_stream
                    for i in range(iters):
                        launch(i, cst)
                graph.replay()
                torch.cuda.synchronize()
                e0.record()
                graph.replay()
                e1.record()
                torch.cuda.synchronize()
                ms = e0.elapsed_time(e1) / iters
                del graph
            except Exception:      # capture not possible: keep the host-loop figure
                pass
            bytes_alg = wbytes + 4 * N + 2 * M * K + 2 * M * N
            gbs = bytes_alg / (ms * 1e-3) / 1e9
            tflops = 2.0 * M * K * N / (ms * 1e-3) / 1e12
            rows.append({'K': K, 'N': N, 'M': M, 'us': ms * 1e3, 'us_host_loop': ms_loop * 1e3, 'GBps': gbs, 'hbm_frac': gbs / hbm,
                        'TFLOPs': tflops, 'tensor_frac': tflops / tf, 'triton_ref_us': ref_us.get((K, N, M))})
        if not cases:
            # the backward product x (M x N) @ W^T -> (M x K), M = 2048 (kernel.py:142-253)
            M = 2048
            xt = torch.randn((M, N), generator=gen, device=dev).half()
            need = _lib.lib.jgq_w4_matmul_workspace_bytes(M, N, K, _lib.W4_TRANSPOSE_B)
            ws = torch.zeros(max(need, 1), dtype=torch.uint8, device=dev)
            out = torch.empty((M, K), dtype=torch.float16, device=dev)
            st = torch.cuda.current_stream().cuda_stream
            def launch_t(i):
                _lib.check(_lib.lib.jgq_w4_matmul(xt.data_ptr(), _lib.F16, packed[i % nbuf].data_ptr(), zero.data_ptr(),
                                                  scale.data_ptr(), _lib.F16, out.data_ptr(), M, N, K, _lib.W4_TRANSPOSE_B,
                                                  ws.data_ptr(), need, st))
            for i in range(2):
                launch_t(i)
            torch.cuda.synchronize()
            e0.record()
            for i in range(3):
                launch_t(i)
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1) / 3
            tflops = 2.0 * M * K * N / (ms * 1e-3) / 1e12
            rows.append({'K': K, 'N': N, 'M': M, 'transpose_b': True, 'us': ms * 1e3, 'TFLOPs': tflops, 'tensor_frac': tflops / tf})
        del packed, qms
        torch.cuda.empty_cache()
    return rows


def bench_w4_sharded(torch, dist, dev, rank, world, peaks):
    """Config-3's largest weight sharded over output channels: every rank multiplies the replicated
    activations by its own (K/2, N/G) slab; with `gather` the (M, N/G) outputs are all-gathered."""
    from jax_gptq_b200 import _lib
    from jax_gptq_b200 import dist as D
    K, N = 8192, 28672
    c0, c1 = D.shard_range(N, rank, world, 128)
    Nl = c1 - c0
    gen = torch.Generator(device=dev).manual_seed(3003 + rank)
    nbuf = max(2, -(-(300 << 20) // (K * Nl // 2)))
    packed = [torch.randint(0, 256, (K // 2, Nl), generator=gen, device=dev, dtype=torch.uint8) for _ in range(nbuf)]
    scale = (0.001 + 0.019 * torch.rand(Nl, generator=gen, device=dev)).half()
    zero = torch.randint(0, 16, (Nl,), generator=gen, device=dev).half()
    rows = []
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for M in (1, 2048):
        x = torch.randn((M, K), generator=torch.Generator(device=dev).manual_seed(5), device=dev).half()
        need = _lib.lib.jgq_w4_matmul_workspace_bytes(M, Nl, K, 0)
        ws = torch.zeros(max(need, 1), dtype=torch.uint8, device=dev)
        out = torch.empty((M, Nl), dtype=torch.float16, device=dev)
        full = torch.empty((world, M, Nl), dtype=torch.float16, device=dev)
        st = torch.cuda.current_stream().cuda_stream
        iters = 20 if M == 1 else 3

        def launch(i):
            _lib.check(_lib.lib.jgq_w4_matmul(x.data_ptr(), _lib.F16, packed[i % nbuf].data_ptr(), zero.data_ptr(),
                                              scale.data_ptr(), _lib.F16, out.data_ptr(), M, Nl, K,
                                              _lib.W4_WEIGHTS_SETTLED, ws.data_ptr(), need, st))
        res = {}
        for gather in (False, True):
            for i in range(3):
                launch(i)
                if gather:
                    dist.all_gather_into_tensor(full, out)
            torch.cuda.synchronize()
            dist.barrier()
            e0.record()
            for i in range(iters):
                launch(i)
                if gather:
                    dist.all_gather_into_tensor(full, out)
            e1.record()
            torch.cuda.synchronize()
            t = torch.tensor([e0.elapsed_time(e1) / iters], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            res['us_with_gather' if gather else 'us_local'] = float(t.item()) * 1e3
        bytes_alg = K * N // 2 + 4 * N + 2 * M * K + 2 * M * N
        rows.append({'K': K, 'N': N, 'M': M, 'n_gpus': world, 'columns_per_rank': Nl, **res,
                     'aggregate_GBps_local': bytes_alg / (res['us_local'] * 1e-6) / 1e9,
                     'aggregate_TFLOPs_local': 2.0 * M * K * N / (res['us_local'] * 1e-6) / 1e12,
                     'timing': 'host loop of launches (max over ranks); the gather is one NCCL all-gather per product'})
    return rows


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--gpus', type=int, default=1)
    ap.add_argument('--steps', type=int, default=3)
    ap.add_argument('--warmup', type=int, default=3)
    ap.add_argument('--impl', default='ours', choices=['ours', 'reference'])
    ap.add_argument('--layers', type=int, default=N_LAYERS, help='blocks to quantize (12 = the full workload)')
    ap.add_argument('--skip-matmul', action='store_true')
    ap.add_argument('--streams', type=int, default=12, help='independent linears in flight (compute streams)')
    ap.add_argument('--no-hessian-stream', action='store_true',
                    help='issue every Hessian GEMM on its linear\'s own stream instead of one lower-priority stream')
    ap.add_argument('--only-matmul', action='store_true', help='run only the packed-int4 matmul sweep')
    ap.add_argument('--matmul-shapes', default='', help='comma list of KxNxM cases for --only-matmul')
    ap.add_argument('--no-settled', action='store_true',
                    help='matmul sweep without JGQ_W4_WEIGHTS_SETTLED (no weight fetch ahead of the previous kernel\'s end)')
    ap.add_argument('--workload', default='gpt2-small', choices=['gpt2-small'] + sorted(SIZED),
                    help='gpt2-small (the headline configuration) or one of the sized configurations')
    ap.add_argument('--skip-cpu', action='store_true')
    ap.add_argument('--skip-parity', action='store_true', help='do not run the oracle comparison of block 0')
    args = ap.parse_args()
    if args.only_matmul:
        import torch
        import jax_gptq_b200 as G
        torch.cuda.set_device(0)
        peaks = {}
        try:
            peaks = json.load(open(os.path.join(ROOT, 'MEASURED_PEAKS.json')))
        except (OSError, ValueError):
            pass
        cases = [tuple(int(v) for v in c.split('x')) for c in args.matmul_shapes.split(',') if c]
        print(json.dumps({'w4_matmul': bench_w4(torch, G, torch.device('cuda', 0), peaks, cases or None,
                                                no_settled=args.no_settled)}), flush=True)
    elif args.impl == 'reference':
        run_reference(args)
    elif args.workload != 'gpt2-small':
        run_sized(args)
    else:
        run_ours(args)


if __name__ == '__main__':
    main()
