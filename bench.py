#!/usr/bin/env python3
"""Headline benchmark: GPT-162M training step (bf16 storage, f32 masters, AdamW) through the persistent executor.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--model gpt_162m]

One "step" = one optimizer step on a micro-batch of 8 x 1024 tokens per GPU: the whole forward + backward + clip + AdamW
task graph run by one launch of the persistent kernel.  Prints ONE JSON line (rank 0).  `value` is micro-batch steps per
second summed over GPUs with the token stream resident in HBM; `e2e` is the same through the C ABI with the step's tokens
copied from pinned host memory and the loss read back inside the timed region.  The `--impl reference` arm (and the
`cpu_baseline` object) time the CPU oracle, a numpy restatement of the reference's op semantics, on a bounded sample.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

PEAK_FALLBACK = {'hbm_gbs': 6650.0, 'bf16_tflops': 1590.0, 'bf16_tflops_sustained': 1400.0}


def peaks():
    p = ROOT / 'MEASURED_PEAKS.json'
    if p.exists():
        return json.loads(p.read_text()), 'measured'
    return dict(PEAK_FALLBACK), 'fallback'


def algorithmic_flops(cfg):
    """Per micro-batch step: GEMM 6 * matmul-params * tokens, attention 3.5 * (4 * B * H * T^2 * hd / 2) per layer."""
    d, F, V, L, N = cfg.d_model, cfg.d_ff, cfg.vocab, cfg.layers, cfg.tokens
    mat = L * (4 * d * d + 2 * d * F) + d * V
    gemm = 6.0 * mat * N
    attn = 3.5 * L * (4.0 * cfg.batch * cfg.heads * cfg.seq * cfg.seq * (d // cfg.heads) / 2)
    return gemm, attn


def task_flops(bundle):
    """Algorithmic FLOPs of every task (GEMM tiles and attention blocks; 0 for the memory-bound ops)."""
    t, a = bundle.tasks, bundle.args
    out = np.zeros(len(t))
    for op, tm, tn in ((122, 128, 256), (34, 64, 64), (114, 64, 64)):
        idx = np.flatnonzero(t['op_id'] == op)
        if len(idx):
            w = a[t['args_off'][idx][:, None] + np.arange(13)[None, :]]
            m = np.minimum(tm, w[:, 8] - w[:, 6]).astype(np.float64)
            n = np.minimum(tn, w[:, 9] - w[:, 7]).astype(np.float64)
            out[idx] = 2.0 * m * n * w[:, 10]
    for op, q0i, Ti, hdi, f in ((45, 7, 8, 11, 4.0), (47, 9, 10, 13, 8.0), (48, 10, 11, 13, 8.0)):
        idx = np.flatnonzero(t['op_id'] == op)
        if len(idx):
            w = a[t['args_off'][idx][:, None] + np.arange(15 if op != 45 else 13)[None, :]]
            q0, T, hd = w[:, q0i].astype(np.float64), w[:, Ti].astype(np.float64), w[:, hdi].astype(np.float64)
            rows = np.minimum(128, T - q0)
            keys = (q0 + rows / 2) if op != 48 else (T - q0 - rows / 2)
            out[idx] = f * rows * keys * hd / 2 * (1.0 if op == 45 else 1.25)
    return out


class ClockSampler:
    """nvidia-smi clocks / throttle reasons sampled every 200 ms while the timed region runs."""
    Q = 'index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,' \
        'clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap'

    def __init__(self, device):
        self.device, self.rows, self.proc = device, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(['nvidia-smi', f'--query-gpu={self.Q}', '--format=csv,noheader,nounits', '-lms', '200', '-i', str(self.device)],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(',')])

    def __exit__(self, *a):
        if self.proc:
            time.sleep(0.25)
            self.proc.terminate()

    def summary(self):
        sm = [float(r[1]) for r in self.rows if len(r) >= 9 and r[1].replace('.', '').isdigit()]
        mx = [float(r[2]) for r in self.rows if len(r) >= 9 and r[2].replace('.', '').isdigit()]
        reasons = set()
        for r in self.rows:
            if len(r) >= 9:
                for name, v in zip(('hw_slowdown', 'hw_thermal_slowdown', 'sw_thermal_slowdown', 'sw_power_cap'), r[5:9]):
                    if v.lower().startswith('active'):
                        reasons.add(name)
        return {'sm_mhz': float(np.median(sm)) if sm else None, 'sm_max_mhz': max(mx) if mx else None, 'reasons': sorted(reasons), 'samples': len(sm)}


def get_bundle(model, rank, world, stream_steps, over):
    """The one-step training bundle of `model` (generated once per box, cached on local disk)."""
    from kvm_b200.bundle import load_bundle
    from kvm_b200.workloads.gpt import build_training, preset
    cfg = preset(model, **over)
    key = f'{model}-r{rank}w{world}-s{stream_steps}-' + '-'.join(f'{k}{v}' for k, v in sorted(over.items()))
    d = Path(tempfile.gettempdir()) / 'kvm_b200_bundles' / key
    if (d / 'metadata.json').exists():
        try:
            return cfg, load_bundle(d)
        except Exception:
            pass
    b = build_training(cfg, 1, rank=rank, world=world, stream_steps=stream_steps).to_bundle(check=False)
    try:
        tmp = d.with_name(d.name + f'.tmp{os.getpid()}')
        b.write(tmp)
        os.replace(tmp, d)
        b.data_dir = d
    except OSError:
        pass
    return cfg, b


def cpu_sample(bundle, cfg, seconds, threads=None):
    """Estimate the CPU oracle's time for one step from a bounded, stratified sample: for every op kind in the bundle a few of
    its tasks (seeded choice) are executed on zero-filled buffers and timed; step time = sum over kinds of count x mean."""
    from oracle.vm_np import VM
    vm = VM(bundle, exact_matmul=False, lazy=True, zeros=True)
    step = vm.buffer('opt_step')
    step.a[:] = 1                       # AdamW wants a 1-based step; the token window must stay inside the stream
    ops = bundle.tasks['op_id']
    kinds = [int(k) for k in np.unique(ops) if k != 0]
    rng = np.random.default_rng(0)
    budget = seconds / max(len(kinds), 1)
    total, ran, t_begin = 0.0, 0, time.perf_counter()
    for k in kinds:
        idx = np.flatnonzero(ops == k)
        pick = rng.permutation(idx)
        spent, n, t_kind = 0.0, 0, time.perf_counter()
        for i in pick[:64]:
            vm.run_task(int(i))         # first execution faults the zero pages in (allocation, not op cost); the second is timed
            t0 = time.perf_counter()
            vm.run_task(int(i))
            spent += time.perf_counter() - t0
            n += 1
            if time.perf_counter() - t_kind > budget:
                break
        total += spent / n * len(idx)
        ran += n
        step.a[:] = 1
    return {'steps_per_s': 1.0 / total, 'seconds': time.perf_counter() - t_begin, 'tasks': ran, 'of_tasks': int(len(ops)), 'kinds': len(kinds)}


def run_reference(args, rank, world):
    """--impl reference: the reference's CPU implementation of the path (the oracle port), all host threads numpy's BLAS takes."""
    if rank != 0:
        return
    cfg, bundle = get_bundle(args.model, 0, 1, 2, {})
    cores = os.cpu_count() or 1
    per = max(2.0, min(20.0, 60.0 / max(args.steps + args.warmup, 1)))
    for _ in range(args.warmup):
        cpu_sample(bundle, cfg, min(per, 3.0))
    vals = [cpu_sample(bundle, cfg, per) for _ in range(args.steps)]
    v = float(np.mean([x['steps_per_s'] for x in vals]))
    sample = f"{vals[-1]['tasks']} of {vals[-1]['of_tasks']} tasks of one step, a few of each of its {vals[-1]['kinds']} op kinds, {vals[-1]['seconds']:.1f} s; step time = sum over kinds of count x mean task time"
    print(json.dumps({
        'impl': 'reference', 'metric': 'gpt162m_train_steps_per_s', 'value': v, 'unit': 'steps/s', 'n_gpus': args.gpus, 'steps': args.steps,
        'warmup': args.warmup, 'ms_per_step': 1000.0 / v, 'higher_is_better': True, 'scaling': 'weak', 'vs_baseline': None, 'dtype': 'bf16',
        'data': 'synthetic', 'config': {'workload': f'{args.model} training step, micro-batch {cfg.batch}x{cfg.seq} tokens, CPU oracle (numpy port of the reference ops)'},
        'cpu_baseline': {'value': v, 'unit': 'steps/s', 'cores': cores, 'kind': 'port', 'sample': sample},
        'e2e': {'value': v, 'unit': 'steps/s', 'h2d_bytes_per_step': 0, 'd2h_bytes_per_step': 0}, 'gpu_launches': 0}))


def run_ours(args, rank, world, local_rank):
    import torch
    import torch.distributed as dist
    from kvm_b200 import build
    from kvm_b200.executor import Executor
    if world > 1:
        dist.init_process_group('nccl', device_id=torch.device('cuda', local_rank))
    if rank == 0:
        build.build()
    if world > 1:
        dist.barrier()
    torch.cuda.set_device(local_rank)
    total = args.warmup + args.steps
    stream_steps = 2 * total + 2
    cfg, bundle = get_bundle(args.model, rank, world, stream_steps, {})
    ex = Executor(device=local_rank)
    ex.load(bundle)
    N = cfg.tokens
    gemm_fl, attn_fl = algorithmic_flops(cfg)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident arm: tokens already in HBM (the stream buffers), no host copies inside the timed region
    ex.run_steps(args.warmup)
    barrier()
    with ClockSampler(local_rank) as clk:
        res = ex.run_steps(args.steps)
        barrier()
    ms = torch.tensor([res.ms], dtype=torch.float64, device='cuda')
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms_total = float(ms.item())
    value = world * args.steps / (ms_total / 1e3)
    loss = float(ex.read_buffer('loss.0')[0, 0])

    # ---- end-to-end arm: the step's tokens come from pinned host memory, the loss goes back, every step
    ids_all, tgt_all = (ex.read_buffer('stream_ids').reshape(-1), ex.read_buffer('stream_tgt').reshape(-1))
    pin_ids = torch.from_numpy(ids_all.copy()).pin_memory()
    pin_tgt = torch.from_numpy(tgt_all.copy()).pin_memory()
    step0 = int(ex.read_buffer('opt_step')[0, 0])
    host_loss = np.zeros(2, np.float32)
    import ctypes as C

    def e2e_step(s):
        lo = (step0 + s) * N
        ex._check(ex.L.kvm_write_buffer(ex._h, ex.index('stream_ids'), pin_ids[lo:lo + N].data_ptr(), N * 4, lo * 4))
        ex._check(ex.L.kvm_write_buffer(ex._h, ex.index('stream_tgt'), pin_tgt[lo:lo + N].data_ptr(), N * 4, lo * 4))
        ex.run()
        ex._check(ex.L.kvm_read_buffer_raw(ex._h, ex.index('loss.0'), host_loss.ctypes.data, 8, 0))
        return float(host_loss[0])

    for s in range(args.warmup):
        e2e_step(s)
    barrier()
    t0 = time.perf_counter()
    for s in range(args.steps):
        e2e_loss = e2e_step(args.warmup + s)
    barrier()
    dt = torch.tensor([time.perf_counter() - t0], dtype=torch.float64, device='cuda')
    if world > 1:
        dist.all_reduce(dt, op=dist.ReduceOp.MAX)
    e2e_value = world * args.steps / float(dt.item())

    if rank == 0:
        pk, pk_kind = peaks()
        kernel_ms = ms_total / args.steps
        achieved = (gemm_fl + attn_fl) / (kernel_ms / 1e3) / 1e12
        peak = pk.get('bf16_tflops_sustained', PEAK_FALLBACK['bf16_tflops_sustained'])
        cpu = cpu_sample(bundle, cfg, args.cpu_seconds) if args.cpu_seconds > 0 else None
        workers, threads, smem = ex.launch_info()
        line = {
            'metric': 'gpt162m_train_steps_per_s', 'value': value, 'unit': 'steps/s', 'n_gpus': world, 'steps': args.steps, 'warmup': args.warmup,
            'ms_per_step': kernel_ms, 'higher_is_better': True, 'scaling': 'weak', 'vs_baseline': None, 'dtype': 'bf16', 'data': 'synthetic',
            'config': {'workload': f'{args.model} training step: {cfg.layers}L d{cfg.d_model} H{cfg.heads} F{cfg.d_ff} V{cfg.vocab} T{cfg.seq}, micro-batch {cfg.batch} per GPU, '
                                   f'bf16 storage + f32 masters, AdamW; one persistent-kernel launch per step ({len(bundle.tasks)} tasks, {len(bundle.succ)} edges)',
                       'tokens_per_step_per_gpu': N, 'parallelism': f'dp{world}', 'l2': 'per-step working set (> 6 GB) exceeds the 126 MB L2',
                       'tc_tasks': ex.tc_task_count(), 'workers': workers, 'threads_per_cta': threads, 'smem_bytes': smem, 'loss_last_step': loss},
            'e2e': {'value': e2e_value, 'unit': 'steps/s', 'h2d_bytes_per_step': 2 * N * 4, 'd2h_bytes_per_step': 8, 'loss': e2e_loss},
            'gpu_launches': 3 * args.steps,
            'clocks': clk.summary(),
            'roofline': {'bound': 'tensor', 'achieved': achieved, 'peak': peak, 'unit': 'TFLOP/s', 'frac': achieved / peak, 'traffic': None,
                         'peak_source': f'{pk_kind} bf16_tflops_sustained', 'flops_per_launch': gemm_fl + attn_fl},
        }
        if cpu:
            line['cpu_baseline'] = {'value': cpu['steps_per_s'], 'unit': 'steps/s', 'cores': os.cpu_count() or 1, 'kind': 'port',
                                    'sample': f"{cpu['tasks']} of {cpu['of_tasks']} tasks of one step, a few of each of its {cpu['kinds']} op kinds, {cpu['seconds']:.1f} s on the numpy oracle; step time = sum over kinds of count x mean task time"}
        print(json.dumps(line))
    ex.close()
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--gpus', type=int, default=1)
    ap.add_argument('--steps', type=int, default=10)
    ap.add_argument('--warmup', type=int, default=3)
    ap.add_argument('--impl', default='ours', choices=['ours', 'reference'])
    ap.add_argument('--model', default='gpt_162m')
    ap.add_argument('--cpu-seconds', type=float, default=15.0, help='length of the CPU-oracle sample behind cpu_baseline (0 = skip)')
    args = ap.parse_args()
    rank, world, local_rank = int(os.environ.get('RANK', 0)), int(os.environ.get('WORLD_SIZE', 1)), int(os.environ.get('LOCAL_RANK', 0))
    args.warmup = max(args.warmup, 3) if args.impl == 'ours' else args.warmup
    if args.impl == 'reference':
        run_reference(args, rank, world)
    else:
        run_ours(args, rank, world, local_rank)


if __name__ == '__main__':
    main()
