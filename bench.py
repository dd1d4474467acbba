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
    # attention: rows x keys score elements (causal: keys up to the row), 4 FLOPs each forward (QK^T and PV) and 10 backward (2.5x,
    # the recomputed scores counted once), split evenly over the dq and dkv tasks
    for op, q0i, Ti, hdi, f in ((45, 7, 8, 11, 4.0), (47, 9, 10, 13, 5.0), (48, 10, 11, 13, 5.0)):
        idx = np.flatnonzero(t['op_id'] == op)
        if len(idx):
            w = a[t['args_off'][idx][:, None] + np.arange(15 if op != 45 else 13)[None, :]]
            q0, T, hd = w[:, q0i].astype(np.float64), w[:, Ti].astype(np.float64), w[:, hdi].astype(np.float64)
            rows = np.minimum(128, T - q0)
            keys = (q0 + rows / 2) if op != 48 else (T - q0 - rows / 2)
            out[idx] = f * rows * keys * hd
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


def workload_name(model, cfg):
    """The configuration both arms name: BASELINE configs[2] for gpt_162m."""
    return (f'{model} training step: {cfg.layers}L d{cfg.d_model} H{cfg.heads} F{cfg.d_ff} V{cfg.vocab} T{cfg.seq}, micro-batch {cfg.batch} x {cfg.seq} tokens per GPU, '
            f'bf16 storage + f32 masters, AdamW lr {cfg.lr} wd {cfg.wd}, seeded weights N(0, {cfg.init_std}), uniform tokens')


# dram__bytes_read.sum + dram__bytes_write.sum of one kvm_exec_kernel launch of the step, from the one-pass ncu captures summarised
# in profiles/bench_gpt162m_launch_list.md (full size) and profiles/kvm_exec_kernel_gpt162m_2l_ncu_full.md (two-layer cut)
DECODE_TRAFFIC_RATIO = (2901808000 + 218917888) / 2855e6      # kvm_static_kernel on qwen3_8b_4l: profiles/kvm_static_kernel_decode_4l_ncu.md
DRAM_TRAFFIC = {'gpt_162m': 24079402496 + 11409903104, 'gpt_162m_2l': 6419808000 + 3092519000}


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
    its tasks (seeded choice) are executed on stand-in values and timed; step time = sum over kinds of count x mean."""
    from oracle.vm_np import VM
    vm = VM(bundle, exact_matmul=False, lazy=True, zeros=_stand_in_values())
    step = vm.buffer('opt_step')
    step.a[:] = 1                       # AdamW wants a 1-based step; the token window must stay inside the stream
    ops = bundle.tasks['op_id']
    kinds = [int(k) for k in np.unique(ops) if k != 0]
    rng = np.random.default_rng(0)
    per_kind = seconds / max(len(kinds), 1)
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
            if time.perf_counter() - t_kind > per_kind:
                break
        total += spent / n * len(idx)
        ran += n
        step.a[:] = 1
    return {'steps_per_s': 1.0 / total, 'seconds': time.perf_counter() - t_begin, 'tasks': ran, 'of_tasks': int(len(ops)), 'kinds': len(kinds)}


def _stand_in_values():
    """Stand-in buffer contents for the bounded CPU sample: ordinary N(0, 0.02) values cut from one shared block instead of zeros
    (exp / tanh / rounding then see ordinary operands), made when a task first touches the buffer.  Materialising the real seeded
    values of a 162M model costs a minute of numpy, which is what the `--impl reference` arm spends; this sample must not."""
    rng = np.random.default_rng(123)
    pool = rng.standard_normal(1 << 24, dtype=np.float32) * np.float32(0.02)

    def make(spec):
        n, shape = spec['rows'] * spec['cols'], (spec['rows'], spec['cols'])
        if spec['dtype'] == 1:
            return np.zeros(shape, np.int32)
        a = np.resize(pool, n).reshape(shape) if n > len(pool) else pool[:n].reshape(shape).copy()
        if spec['name'].startswith('v.'):
            a = np.abs(a)                                      # second moments are non-negative
        if spec['dtype'] == 2:
            from oracle.ops_np import bf16_round
            a = bf16_round(a)
        return np.ascontiguousarray(a)
    return make


def cpu_real_step(bundle, limit_s):
    """ONE real step of the CPU oracle on the bench's own bundle (seeded weights, the same token stream), all host threads numpy's
    BLAS takes.  Only the step is timed, not the creation of the buffers.  If the box is so slow that the step passes `limit_s`,
    the run stops there and the step time is extrapolated from the share of tasks done (said so in the result)."""
    from oracle.vm_np import VM
    t0 = time.perf_counter()
    vm = VM(bundle, exact_matmul=False)
    t_init = time.perf_counter() - t0
    t0 = time.perf_counter()
    vm.run(time_limit=limit_s)
    dt = time.perf_counter() - t0
    done, nt = int(vm.exec_count.sum()), len(bundle.tasks)
    loss = float(vm.buffer('loss.0').a[0, 0]) if done == nt else None
    return {'seconds': dt * nt / max(done, 1), 'measured_seconds': dt, 'tasks': done, 'of_tasks': nt, 'init_seconds': t_init, 'loss': loss}


def run_reference(args, rank, world):
    """--impl reference: the reference's CPU implementation of the path (the oracle port), all host threads numpy's BLAS takes."""
    if rank != 0:
        return
    cfg, bundle = get_bundle(args.model, 0, 1, 2, {})
    cores = os.cpu_count() or 1
    # One REAL step is timed (about a minute of CPU work on this model, plus as much again to create the seeded buffers): that is
    # the bounded sample.  `steps` in the line is the number of steps actually executed and timed, so ms_per_step x steps is the
    # CPU time this run really spent in the timed region; the requested K / W are echoed beside it.
    r = cpu_real_step(bundle, args.cpu_step_limit)
    v = 1.0 / r['seconds']
    whole = r['tasks'] == r['of_tasks']
    sample = (f"one real step of the numpy oracle on the bench's own bundle ({r['of_tasks']} tasks, seeded weights and tokens), {r['measured_seconds']:.1f} s timed"
              + ('' if whole else f", stopped after {r['tasks']} tasks at the time limit and extrapolated by task count")
              + f"; creating the buffers took {r['init_seconds']:.1f} s more (untimed); requested steps {args.steps}, warmup {args.warmup}: not repeated on the CPU")
    print(json.dumps({
        'impl': 'reference', 'metric': 'gpt162m_train_steps_per_s', 'value': v, 'unit': 'steps/s', 'n_gpus': args.gpus, 'steps': 1, 'steps_requested': args.steps,
        'warmup': 0, 'warmup_requested': args.warmup, 'ms_per_step': 1000.0 / v, 'higher_is_better': True, 'scaling': 'weak', 'vs_baseline': None, 'dtype': 'bf16',
        'data': 'synthetic', 'config': {'workload': workload_name(args.model, cfg), 'tokens_per_step_per_gpu': cfg.tokens, 'parallelism': f'dp{args.gpus}',
                                        'engine': 'CPU oracle: numpy port of the reference ops, all host threads BLAS takes', 'loss': r['loss']},
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
            'config': {'workload': workload_name(args.model, cfg), 'tokens_per_step_per_gpu': N, 'parallelism': f'dp{world}',
                       'engine': f'one persistent-kernel launch per step ({len(bundle.tasks)} tasks, {len(bundle.succ)} edges)',
                       'l2': 'per-step working set (> 6 GB) exceeds the 126 MB L2',
                       'tc_tasks': ex.tc_task_count(), 'workers': workers, 'threads_per_cta': threads, 'smem_bytes': smem, 'loss_last_step': loss},
            'e2e': {'value': e2e_value, 'unit': 'steps/s', 'h2d_bytes_per_step': 2 * N * 4, 'd2h_bytes_per_step': 8, 'loss': e2e_loss},
            'gpu_launches': 3 * args.steps,
            'clocks': clk.summary(),
            'roofline': {'bound': 'tensor', 'achieved': achieved, 'peak': peak, 'unit': 'TFLOP/s', 'frac': achieved / peak, 'traffic': DRAM_TRAFFIC.get(args.model),
                         'peak_source': f'{pk_kind} bf16_tflops_sustained', 'flops_per_launch': gemm_fl + attn_fl},
        }
        ex.close()
        try:
            line['busy'] = trace_split(bundle, local_rank)
        except Exception as e:
            line['busy'] = {'error': str(e)[:300]}
        extras = set(args.extras.split(',')) if world == 1 else set()
        for key, name, fn in (('decode', 'decode', lambda: run_decode(args, local_rank)), ('alone', 'kernels_alone', lambda: run_alone(local_rank)),
                              ('small', 'small_models', lambda: run_small(local_rank)), ('355m', 'gpt_355m', lambda: run_355m(local_rank))):
            if key not in extras or (key == 'decode' and args.decode_tokens <= 0):
                continue
            try:
                line[name] = fn()
            except Exception as e:      # the training line stands on its own
                line[name] = {'error': str(e)[:300]}
        if cpu:
            line['cpu_baseline'] = {'value': cpu['steps_per_s'], 'unit': 'steps/s', 'cores': os.cpu_count() or 1, 'kind': 'port',
                                    'sample': f"{cpu['tasks']} of {cpu['of_tasks']} tasks of one step, a few of each of its {cpu['kinds']} op kinds, {cpu['seconds']:.1f} s on the numpy oracle; step time = sum over kinds of count x mean task time"}
        print(json.dumps(line))
    ex.close()
    if world > 1:
        dist.destroy_process_group()


OP_FAMILY = {122: 'gemm_tc', 34: 'gemm_f32', 114: 'gemm_f32', 45: 'attention', 46: 'attention', 47: 'attention', 48: 'attention', 35: 'norm', 37: 'norm', 39: 'norm',
             61: 'colsum', 127: 'cross_entropy', 52: 'cross_entropy', 54: 'adamw', 55: 'gradnorm', 56: 'gradnorm', 113: 'round_bf16', 41: 'gelu_bwd', 32: 'embedding',
             33: 'embedding', 0: 'noop', 62: 'plumbing', 60: 'plumbing'}


def trace_split(bundle, device, flags=0):
    """ONE traced step, outside every timed region: the fraction of worker time spent inside tasks (sum(end - start) /
    (workers x span), the reference's formula, results/2026-11-11-162m-ceiling/README.md:50-56) and its split by op family."""
    from kvm_b200.executor import Executor
    with Executor(device=device, trace=True, flags=flags) as ex:
        ex.load(bundle)
        ex.run()
        res = ex.run()
        st, en, _ = ex.trace()
        workers = ex.launch_info()[0]
    ok = (en > st) & (st > 0)
    span = float(en[ok].max() - st[ok].min())
    dur = (en - st).astype(np.float64) * ok
    fam = {}
    for op in np.unique(bundle.tasks['op_id']):
        sel = bundle.tasks['op_id'] == op
        name = OP_FAMILY.get(int(op), f'op{int(op)}')
        fam[name] = fam.get(name, 0.0) + float(dur[sel].sum())
    return {'busy_frac': float(dur.sum() / (workers * span)), 'busy_frac_by_family': {k: round(v / (workers * span), 4) for k, v in sorted(fam.items(), key=lambda kv: -kv[1])},
            'idle_frac': float(1.0 - dur.sum() / (workers * span)), 'traced_step_ms': res.ms, 'span_ms': span / 1e6, 'workers': workers,
            'note': 'one traced step after the timed region (tracing adds two timestamps and a store per task)'}


def run_dp(args, rank, world, local_rank):
    """N > 1: data-parallel training, weak scaling (every rank keeps the micro-batch of 8 x 1024 tokens), in two forms:
      fused   ONE launch per step and rank; the gradient all-reduce is tasks of the graph (peer stores into the other ranks' arenas and
              inboxes over NVLink, flag words, bounded waits) that run while the backward still has work;
      nccl    backward launch -> one NCCL all-reduce (mean) over the gradient arena -> optimizer launch.
    Both are measured (KVM_B200_DP=fused|nccl picks one); the line's value is the faster form whose replicas ended equal."""
    import torch
    import torch.distributed as dist
    from kvm_b200 import build
    from kvm_b200.dp import DataParallelStep, DataParallelStepFused, grad_arena_layout
    from kvm_b200.workloads.gpt import build_training, preset
    dist.init_process_group('nccl', device_id=torch.device('cuda', local_rank))
    torch.cuda.set_device(local_rank)
    if rank == 0:
        build.build()
    dist.barrier()
    cfg = preset(args.model)
    total = args.warmup + args.steps

    def exchange_handles(mine):
        out = [None] * world
        dist.all_gather_object(out, mine)
        return out

    def measure(form):
        comm_ms = []
        if form == 'fused':
            dp = DataParallelStepFused(cfg, rank, world, local_rank, total + 1, exchange_handles)
            n_arena = dp.arena_elems
            step = lambda: (dp.step(),)
        else:
            g = build_training(cfg, 1, rank=rank, world=world, stream_steps=total + 1)
            bundles = g.to_bundles_split(g.split_at)
            _, n_arena = grad_arena_layout(bundles[0])
            arena = torch.zeros(n_arena, dtype=torch.float32, device='cuda')
            dp = DataParallelStep(cfg, rank, world, local_rank, arena.data_ptr(), total + 1, bundles=bundles)
            ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

            def all_reduce_mean():
                ev0.record()
                dist.all_reduce(arena, op=dist.ReduceOp.AVG)
                ev1.record()
                torch.cuda.synchronize()
                comm_ms.append(ev0.elapsed_time(ev1))
            step = lambda: dp.step(all_reduce_mean)
        for _ in range(args.warmup):
            torch.cuda.synchronize(); dist.barrier()      # the ranks start a step together (a fused step waits for its peers inside the launch)
            step()
        dist.barrier(); torch.cuda.synchronize()
        comm_ms.clear()
        dev_ms, t0 = 0.0, time.perf_counter()
        with ClockSampler(local_rank) as clk:
            for _ in range(args.steps):
                dev_ms += sum(r.ms for r in step())
            dist.barrier(); torch.cuda.synchronize()
            wall = time.perf_counter() - t0
        dev_ms += sum(comm_ms)
        t = torch.tensor([dev_ms, wall * 1e3], dtype=torch.float64, device='cuda')
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        loss = float(dp.bwd.read_buffer('loss.0')[0, 0])
        w0 = torch.tensor([float(np.abs(dp.bwd.read_buffer('w.lnf.g')).sum())], dtype=torch.float64, device='cuda')
        wmax, wmin = w0.clone(), w0.clone()
        dist.all_reduce(wmax, op=dist.ReduceOp.MAX); dist.all_reduce(wmin, op=dist.ReduceOp.MIN)
        dp.close()
        torch.cuda.empty_cache()
        return {'form': form, 'dev_total': float(t[0]), 'wall_total': float(t[1]), 'loss': loss, 'weights_abs_sum': float(w0), 'replicas_equal': bool(float(wmax) == float(wmin)),
                'allreduce_ms_per_step': float(np.mean(comm_ms)) if comm_ms else None, 'launches_per_step': 3 if form == 'fused' else 6, 'n_arena': n_arena, 'clocks': clk.summary()}

    which = os.environ.get('KVM_B200_DP', 'both')
    runs = {}
    for form in (['fused', 'nccl'] if which == 'both' else [which]):
        try:
            runs[form] = measure(form)
        except Exception as e:
            runs[form] = {'form': form, 'error': str(e)[:300]}
    valid = [r for r in runs.values() if 'error' not in r and r['replicas_equal']] or [r for r in runs.values() if 'error' not in r]
    tp = None
    if args.decode_tokens > 0:
        try:
            tp = run_decode_tp(args, rank, world, local_rank)
        except Exception as e:          # the training line stands on its own
            tp = {'error': str(e)[:300]}
    if rank == 0:
        if not valid:
            print(json.dumps({'metric': 'gpt162m_train_steps_per_s', 'value': None, 'n_gpus': world, 'error': {k: v.get('error') for k, v in runs.items()}, 'decode_tp': tp}))
            dist.destroy_process_group()
            return
        best = min(valid, key=lambda r: r['wall_total'])
        gemm_fl, attn_fl = algorithmic_flops(cfg)
        pk, pk_kind = peaks()
        ms_step = best['dev_total'] / args.steps
        value = world * args.steps / (best['wall_total'] / 1e3)          # host wall clock between barriers: includes launch gaps and the collective
        achieved = (gemm_fl + attn_fl) / (ms_step / 1e3) / 1e12
        peak = pk.get('bf16_tflops_sustained', PEAK_FALLBACK['bf16_tflops_sustained'])
        how = {'fused': f"data parallel, one launch per step and rank: the all-reduce (mean) of {best['n_arena'] * 4 / 1e6:.0f} MB of f32 gradients is tasks of the graph "
                        '(peer stores over NVLink, flag words, bounded waits) overlapped with the backward',
               'nccl': f"data parallel: backward launch, NCCL all-reduce (mean) of {best['n_arena'] * 4 / 1e6:.0f} MB of f32 gradients, optimizer launch"}[best['form']]
        forms = {k: ({'steps_per_s': world * args.steps / (v['wall_total'] / 1e3), 'ms_per_step': v['wall_total'] / args.steps, 'device_ms_per_step': v['dev_total'] / args.steps,
                      'allreduce_ms_per_step': v['allreduce_ms_per_step'], 'replicas_equal': v['replicas_equal'], 'loss_last_step_rank0': v['loss'],
                      'weights_abs_sum_rank0': v['weights_abs_sum']} if 'error' not in v else {'error': v['error']}) for k, v in runs.items()}
        print(json.dumps({
            'metric': 'gpt162m_train_steps_per_s', 'value': value, 'unit': 'steps/s', 'n_gpus': world, 'steps': args.steps, 'warmup': args.warmup,
            'ms_per_step': best['wall_total'] / args.steps, 'higher_is_better': True, 'scaling': 'weak', 'vs_baseline': None, 'dtype': 'bf16', 'data': 'synthetic',
            'config': {'workload': workload_name(args.model, cfg), 'tokens_per_step_per_gpu': cfg.tokens, 'parallelism': f'dp{world}', 'engine': how,
                       'l2': 'per-step working set (> 6 GB) exceeds the 126 MB L2',
                       'device_ms_per_step': ms_step, 'allreduce_ms_per_step': best['allreduce_ms_per_step'], 'loss_last_step_rank0': best['loss'],
                       'replicas_equal': best['replicas_equal'], 'forms': forms},
            'e2e': {'value': value, 'unit': 'steps/s', 'h2d_bytes_per_step': 0, 'd2h_bytes_per_step': 0, 'note': 'multi-GPU arm keeps tokens resident; the 1-GPU line carries the host-copy arm'},
            'gpu_launches': best['launches_per_step'] * args.steps, 'clocks': best['clocks'],
            'roofline': {'bound': 'tensor', 'achieved': achieved, 'peak': peak, 'unit': 'TFLOP/s', 'frac': achieved / peak, 'traffic': None,
                         'peak_source': f'{pk_kind} bf16_tflops_sustained (per GPU, device time incl. all-reduce)'},
            'decode_tp': tp}))
    dist.destroy_process_group()


def tp_parity_tokens(rank, world, device, exchange_handles, ntok=6):
    """The one-launch tensor-parallel form on a small model whose shards are exact slices of the unsharded weights: the greedy tokens
    over the `world` GPUs must equal the tokens of the unsharded graph run on one GPU."""
    import torch
    import torch.distributed as dist
    from kvm_b200.tp import TensorParallelDecodeFused, pick_token
    from kvm_b200.workloads.decode import build_decode, preset
    cfg = preset('decode_tiny', init_std=0.08, kv_heads=max(2, world))          # 8 query heads: up to 8 ranks
    if cfg.heads % world or cfg.kv_heads % world or cfg.ffn % world or cfg.vocab % world:
        return {'skipped': f'decode_tiny does not split over {world} ranks'}
    logits = torch.zeros(1, cfg.vocab // world, dtype=torch.float32, device='cuda')
    tok = torch.full((1, 1), 3 % cfg.vocab, dtype=torch.int32, device='cuda')
    tpd = TensorParallelDecodeFused(cfg, rank, world, device, {'u0.logits': logits.data_ptr(), 'u0.tok': tok.data_ptr()}, exchange_handles, exact=True)
    got = []
    for _ in range(ntok):
        torch.cuda.synchronize(); dist.barrier()
        tpd.ex.run()
        val, idx = logits.max(dim=1)
        allp = torch.zeros(world, 2, dtype=torch.float64, device='cuda')
        dist.all_gather_into_tensor(allp, torch.stack([val.double(), (idx + rank * logits.shape[1]).double()], dim=1))
        t = pick_token((float(a), int(b)) for a, b in allp.cpu().numpy())
        tok.fill_(t)
        got.append(t)
    torch.cuda.synchronize(); dist.barrier()
    tpd.close()
    ref, err = None, None
    if rank == 0:            # the unsharded graph of the same model on this rank's GPU alone (tests/ pin that path to the CPU oracle token by token)
        try:
            from kvm_b200.executor import Executor
            with Executor(device=device) as ex:
                ex.load(build_decode(cfg).to_bundle())
                ref = []
                for _ in range(ntok):
                    ex.run()
                    ref.append(int(ex.read_buffer('u0.tok')[0, 0]))
        except Exception as e:      # the other ranks wait at the barrier below either way
            ref, err = None, str(e)[:200]
    torch.cuda.synchronize(); dist.barrier()
    out = {'model': 'decode_tiny, exact shards', 'tokens': got, 'unsharded_tokens': ref, 'match': None if ref is None else got == ref}
    if err:
        out['error'] = err
    return out


def run_decode_tp(args, rank, world, device):
    """Tensor-parallel greedy decode of the 8B shape over the `world` GPUs (strong scaling: the same token, weights and cache split
    over the ranks), timed with CUDA events around whole tokens, max over ranks.  Default: ONE launch of the persistent kernel per
    token and rank, the two partial sums per layer are tasks (peer stores into the other ranks' inboxes over NVLink, flag release,
    bounded wait: extension ops 302 / 303); only the token choice over the vocabulary slices is a host-side all-gather.
    KVM_B200_TP=segments: 2 * layers + 1 launches per token with an NCCL all-reduce of the [1, hidden] partial between them."""
    import torch
    import torch.distributed as dist
    from kvm_b200.tp import TensorParallelDecode, TensorParallelDecodeFused, pick_token
    from kvm_b200.workloads.decode import kv_bytes, preset, weight_bytes
    cfg = preset(args.decode_model)
    if cfg.heads % world or cfg.kv_heads % world or cfg.ffn % world or cfg.vocab % world:
        return {'error': f'{args.decode_model} does not split over {world} ranks'}
    fused = os.environ.get('KVM_B200_TP', 'fused') != 'segments'
    names = [] if fused else [f'u0.l{l}.{n}' for l in range(cfg.layers) for n in ('x1', 'x2')]
    bufs = {n: torch.zeros(1, cfg.hidden, dtype=torch.float32, device='cuda') for n in names}
    logits = torch.zeros(1, cfg.vocab // world, dtype=torch.float32, device='cuda')
    tok = torch.full((1, 1), 3, dtype=torch.int32, device='cuda')
    bind = {n: t.data_ptr() for n, t in bufs.items()}
    bind.update({'u0.logits': logits.data_ptr(), 'u0.tok': tok.data_ptr()})
    from kvm_b200.executor import CFG_CHAIN

    def exchange_handles(mine):
        out = [None] * world
        dist.all_gather_object(out, mine)
        return out

    if fused:
        tpd = TensorParallelDecodeFused(cfg, rank, world, device, bind, exchange_handles, flags=CFG_CHAIN)
    else:
        tpd = TensorParallelDecode(cfg, rank, world, device, bind, flags=CFG_CHAIN)

    def all_reduce_sum(name):           # first tokens: launches on the handles' own streams, so the host waits for the collective
        dist.all_reduce(bufs[name], op=dist.ReduceOp.SUM)
        torch.cuda.current_stream().synchronize()

    def all_reduce_queued(name):        # timed tokens: everything is queued on one stream, stream order is the only synchronisation
        dist.all_reduce(bufs[name], op=dist.ReduceOp.SUM)

    def choose():
        val, idx = logits.max(dim=1)
        mine = torch.stack([val.double(), (idx + rank * logits.shape[1]).double()], dim=1)      # [1, 2]
        allp = torch.zeros(world, 2, dtype=torch.float64, device='cuda')
        dist.all_gather_into_tensor(allp, mine)
        p = allp.cpu().numpy()
        tok.fill_(pick_token((float(a), int(b)) for a, b in p))
        torch.cuda.current_stream().synchronize()

    parity = None
    if fused:
        try:
            parity = tp_parity_tokens(rank, world, device, exchange_handles)
        except Exception as e:
            parity = {'error': str(e)[:200]}
    step = (lambda: tpd.token(choose)) if fused else (lambda: tpd.token(all_reduce_sum, choose))
    step_async = (lambda: tpd.token_async(choose)) if fused else (lambda: tpd.token_async(all_reduce_queued, choose))
    ntok, warm = min(args.decode_tokens, 32 if fused else 8), 2
    for _ in range(warm):
        torch.cuda.synchronize(); dist.barrier()
        step()
    tpd.use_stream(torch.cuda.current_stream().cuda_stream)
    step_async()
    dist.barrier(); torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(ntok):
        step_async()
    e1.record(); torch.cuda.synchronize()
    kern_ms = sum(tpd.finish())         # kernel time of the last token's launches
    t = torch.tensor([e0.elapsed_time(e1), kern_ms * ntok], dtype=torch.float64, device='cuda')
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    last = int(tok.item())
    nlaunch = 3 * len(tpd.handles)
    tpd.close()
    ms_tok = float(t[0]) / ntok
    pk, kind = peaks()
    bytes_tok = weight_bytes(cfg) + kv_bytes(cfg, cfg.ctx + warm + ntok / 2)
    gbs = bytes_tok / (ms_tok / 1e3) / 1e9
    how = ('one launch per token and rank; the 2 x layers partial sums are tasks: peer stores into the other ranks\' inboxes, flag release, bounded wait'
           if fused else '2 x layers + 1 launches per token with an NCCL all-reduce of the partial between them')
    return {'metric': 'decode_tokens_per_s', 'value': 1e3 / ms_tok, 'unit': 'tok/s', 'scaling': 'strong', 'n_gpus': world, 'ms_per_token': ms_tok,
            'parity': parity, 'kernel_ms_per_token': float(t[1]) / ntok, 'launches_per_token': nlaunch, 'exchanges_per_token': 2 * cfg.layers, 'exchange': how, 'tokens': ntok, 'last_token': last,
            'workload': f'{args.decode_model} batch 1 context {cfg.ctx}, tensor parallel over {world} GPUs (heads / FFN columns / vocabulary split), seeded shards',
            'roofline': {'bound': 'hbm', 'achieved': gbs, 'unit': 'GB/s', 'peak': world * pk.get('hbm_gbs', PEAK_FALLBACK['hbm_gbs']),
                         'frac': gbs / (world * pk.get('hbm_gbs', PEAK_FALLBACK['hbm_gbs'])), 'bytes_per_token': bytes_tok, 'peak_source': f'{kind} hbm_gbs x {world} GPUs'}}


def run_decode(args, device):
    """Second headline: greedy decode of the 8B shape (batch 1, 4K context) through the same executor: tokens/s and the
    fraction of the measured HBM copy bandwidth that the algorithmic bytes per token (bf16 weights + KV cache read) reach."""
    import ctypes as C
    from kvm_b200.executor import Executor
    from kvm_b200.workloads.decode import build_decode, kv_bytes, preset, weight_bytes
    cfg = preset(args.decode_model)
    d = Path(tempfile.gettempdir()) / 'kvm_b200_bundles' / f'decode-{args.decode_model}-b{cfg.batch}-s{cfg.splits}-r{cfg.rows_per_task}-j{cfg.join_threshold}'
    from kvm_b200.bundle import load_bundle
    if (d / 'metadata.json').exists():
        bundle = load_bundle(d)
    else:
        bundle = build_decode(cfg).to_bundle(check=False)
        try:
            bundle.write(d)
        except OSError:
            pass
    ex = Executor(device=device)
    ex.load(bundle)
    ntok, warm = args.decode_tokens, 3
    ex.run_steps(warm)
    path = ex.plan_info()
    res = ex.run_steps(ntok)
    tok_s = ntok / (res.ms / 1e3)
    ctx_mid = cfg.ctx + warm + ntok / 2
    bytes_tok = weight_bytes(cfg) + kv_bytes(cfg, ctx_mid)
    pk, kind = peaks()
    gbs = bytes_tok * tok_s / 1e9
    tok = np.zeros(1, np.int32)
    n_e2e = min(ntok, max(1, cfg.tmax - cfg.ctx - warm - ntok - 8), 64)      # the cache has room for tmax - ctx appended tokens in all
    t0 = time.perf_counter()
    for _ in range(n_e2e):
        ex.run()
        ex._check(ex.L.kvm_read_buffer_raw(ex._h, ex.index('u0.tok'), tok.ctypes.data, 4, 0))
    e2e = n_e2e / (time.perf_counter() - t0)
    out = {'metric': 'decode_tokens_per_s', 'workload': f'{args.decode_model}: {cfg.layers}L hidden {cfg.hidden} {cfg.heads}q/{cfg.kv_heads}kv heads hd{cfg.head_dim} ffn {cfg.ffn} '
                                                      f'vocab {cfg.vocab}, bf16 weights, batch {cfg.batch}, context {cfg.ctx}, greedy; {len(bundle.tasks)} tasks per token, reference op set (the QK-norm variant is timed beside it)',
           'value': tok_s, 'unit': 'tok/s', 'ms_per_token': res.ms / ntok, 'tokens': ntok, 'e2e': {'value': e2e, 'unit': 'tok/s', 'h2d_bytes_per_step': 0, 'd2h_bytes_per_step': 4, 'tokens': n_e2e},
           'roofline': {'bound': 'hbm', 'achieved': gbs, 'peak': pk.get('hbm_gbs', PEAK_FALLBACK['hbm_gbs']), 'unit': 'GB/s', 'frac': gbs / pk.get('hbm_gbs', PEAK_FALLBACK['hbm_gbs']),
                        'bytes_per_token': bytes_tok, 'peak_source': f'{kind} hbm_gbs', 'traffic': bytes_tok * DECODE_TRAFFIC_RATIO,
                        'traffic_note': 'DRAM bytes of the 4-layer cut under ncu (3.12 GB for 2.86 GB algorithmic), scaled by the algorithmic bytes'}, 'last_token': int(tok[0]),
           'path': {'static_schedule': path[0], 'stream_ring': path[1], 'planned_us_per_token': path[2]}}
    ex.close()
    pkh = pk.get('hbm_gbs', PEAK_FALLBACK['hbm_gbs'])
    try:        # Qwen3's per-head QK RMSNorm in front of the rotary embedding (extension op 300; not in the reference op set)
        cfgq = preset(args.decode_model, qk_norm=True)
        with Executor(device=device) as exq:
            exq.load(build_decode(cfgq).to_bundle(check=False))
            exq.run_steps(warm)
            rq = exq.run_steps(min(ntok, 32))
        msq = rq.ms / min(ntok, 32)
        out['qk_norm'] = {'value': 1e3 / msq, 'unit': 'tok/s', 'ms_per_token': msq, 'roofline_frac': bytes_tok / (msq / 1e3) / 1e9 / pkh}
    except Exception as e:
        out['qk_norm'] = {'error': str(e)[:300]}
    try:        # batch 8, two ways: the users as ROWS of shared activation matrices (extension op 301: one pass over the weights per
        #         step), and as 8 independent row users (the reference's op set: every user streams the weights again)
        from kvm_b200.workloads.decode import build_decode_rows
        cfg8 = preset(args.decode_model, batch=8)
        ideal = weight_bytes(cfg8) + 8 * kv_bytes(cfg8, cfg8.ctx + 5)
        out['batch8'] = {}
        for tag, builder in (('rows', build_decode_rows), ('users', build_decode)):
            b8 = builder(cfg8).to_bundle(check=False)
            with Executor(device=device) as ex8:
                ex8.load(b8)
                ex8.run_steps(2)
                r8 = ex8.run_steps(6)
            ms8 = r8.ms / 6
            out['batch8'][tag] = {'value': 8 / (ms8 / 1e3), 'unit': 'tok/s', 'ms_per_step': ms8, 'tasks_per_step': len(b8.tasks),
                                  'roofline': {'bound': 'hbm', 'achieved': ideal / (ms8 / 1e3) / 1e9, 'unit': 'GB/s', 'peak': pkh, 'frac': ideal / (ms8 / 1e3) / 1e9 / pkh,
                                               'bytes_per_step': ideal}}
            del b8
        out['batch8']['note'] = 'algorithmic bytes count the weights once per step and the 8 caches; the independent users stream the weights 8 times'
    except Exception as e:
        out['batch8'] = {'error': str(e)[:300]}
    return out


def run_alone(device):
    """The two dominant op kinds timed alone through the executor (a graph of nothing but independent tasks of that kind, inputs
    larger than L2), to read beside the whole-step numbers: tensor-core GEMM tiles of the three K depths a GPT-162M step has, and
    the streaming GEMV over an LM-head sized weight matrix."""
    from kvm_b200.executor import Executor
    from kvm_b200.workloads.graph import Graph
    pk, kind = peaks()
    out = {}
    sd = lambda n, sc: {'kind': 'seeded', 'seed': n, 'scale': sc, 'dist': 'normal'}
    for name, (M, N, K, flags, reps) in {'gemm_fwd_k768': (8192, 3072, 768, 0, 6), 'gemm_fwd_k3072': (8192, 768, 3072, 0, 8), 'gemm_wgrad_k8192': (3072, 768, 8192, 1, 16)}.items():
        g = Graph('alone')
        for r in range(reps):                 # independent products: operands of their own, so nothing is re-read from L2 by design
            a = g.buffer(f'a{r}', *((K, M) if flags & 1 else (M, K)), 'bf16', sd(3 * r + 1, 1.0))
            b = g.buffer(f'b{r}', K, N, 'bf16', sd(3 * r + 2, 0.02))
            o = g.buffer(f'o{r}', M, N, 'bf16')
            for m0 in range(0, M, 128):
                for n0 in range(0, N, 256):
                    g.task('matmul_mma_bf16', {'a': a, 'b': b, 'out': o, 'bias': None, 'res': None, 'pre': None, 'm0': m0, 'n0': n0, 'M': M, 'N': N, 'K': K, 'flags': flags,
                                               'alpha': 1.0}, [], [(o, (m0, min(m0 + 128, M)), (n0, min(n0 + 256, N)))], 5, f'{r}.{m0}.{n0}')
        bundle = g.to_bundle(check=False)
        with Executor(device=device) as ex:
            ex.load(bundle); ex.run()
            ms = min(ex.run().ms for _ in range(3))
        tf = 2.0 * M * N * K * reps / (ms * 1e-3) / 1e12
        peak = pk.get('bf16_tflops_sustained', PEAK_FALLBACK['bf16_tflops_sustained'])
        out[name] = {'shape': [M, N, K], 'tiles': len(bundle.tasks), 'ms': ms, 'achieved': tf, 'unit': 'TFLOP/s', 'peak': peak, 'frac': tf / peak, 'bound': 'tensor'}
    g = Graph('alone')
    rows, K, ntask = 256, 4096, 148 * 4
    w = g.buffer('w', rows * ntask, K, 'bf16', sd(1, 0.02)); x = g.buffer('x', 1, K, init=sd(2, 1.0)); o = g.buffer('o', 1, rows * ntask)
    for i in range(ntask):
        g.task('gemv_bf16', {'x': x, 'x2': None, 'gamma': None, 'w': w, 'out': o, 'res': None, 'n0': i * rows, 'n1': (i + 1) * rows, 'K': K, 'pro': 0, 'eps': 1e-6},
               [x, (w, (i * rows, (i + 1) * rows))], [(o, (0, 1), (i * rows, (i + 1) * rows))], 5, f't{i}')
    bundle = g.to_bundle(check=False)
    with Executor(device=device) as ex:
        ex.load(bundle); ex.run()
        ms = min(ex.run().ms for _ in range(3))
    gbs = rows * ntask * K * 2 / (ms * 1e-3) / 1e9
    peak = pk.get('hbm_gbs', PEAK_FALLBACK['hbm_gbs'])
    out['gemv_k4096'] = {'shape': [rows * ntask, K], 'tasks': ntask, 'ms': ms, 'achieved': gbs, 'unit': 'GB/s', 'peak': peak, 'frac': gbs / peak, 'bound': 'hbm'}
    out.update(run_alone_more(device, pk))
    out['note'] = f'whole launches (about 17 us of launch, arming and shutdown included); peaks: {kind}'
    return out


def run_alone_more(device, pk):
    """Attention (TFLOP/s) and the memory-bound families (GB/s of their algorithmic bytes) alone, at the GPT-162M step's sizes and
    task granularity: graphs of independent tasks of one kind, operands larger than L2."""
    from kvm_b200.executor import Executor
    from kvm_b200.workloads.gpt import _Emit, preset
    out = {}
    hbm, tfl = pk.get('hbm_gbs', PEAK_FALLBACK['hbm_gbs']), pk.get('bf16_tflops_sustained', PEAK_FALLBACK['bf16_tflops_sustained'])
    cfg = preset('gpt_162m')
    N, d, F, V, T, H = cfg.tokens, cfg.d_model, cfg.d_ff, cfg.vocab, cfg.seq, cfg.heads
    sd = lambda n, sc: {'kind': 'seeded', 'seed': n, 'scale': sc, 'dist': 'normal'}

    def timed(g):
        bundle = g.to_bundle(check=False)
        with Executor(device=device) as ex:
            ex.load(bundle); ex.run()
            return min(ex.run().ms for _ in range(3)), bundle

    def emitter():
        e = _Emit.__new__(_Emit)
        from kvm_b200.workloads.graph import Graph
        e.c, e.g, e.bf, e.act, e.params, e.prio = cfg, Graph('alone'), True, 'bf16', {}, 5
        e.g.join_threshold = cfg.join_threshold
        return e

    # ---- causal attention forward / dq / dkv on bf16 q, k, v (tcgen05 path), 3 independent copies
    reps = 3
    e = emitter(); g = e.g
    for r in range(reps):
        q, k, v, do = (g.buffer(f'{n}{r}', N, d, 'bf16', sd(10 * r + i, 1.0)) for i, n in enumerate(('q', 'k', 'v', 'do')))
        o, lse = g.buffer(f'o{r}', N, d, 'bf16'), g.buffer(f'lse{r}', cfg.batch * H * T, 1)
        e.attention(f'f{r}', q, k, v, o, lse)
    ms, b = timed(g)
    fl = float(task_flops(b).sum())
    out['attention_fwd'] = {'tasks': len(b.tasks), 'ms': ms, 'achieved': fl / (ms * 1e-3) / 1e12, 'unit': 'TFLOP/s', 'peak': tfl, 'frac': fl / (ms * 1e-3) / 1e12 / tfl, 'bound': 'tensor'}
    e = emitter(); g = e.g
    for r in range(reps):
        q, k, v, do, o = (g.buffer(f'{n}{r}', N, d, 'bf16', sd(10 * r + i, 1.0)) for i, n in enumerate(('q', 'k', 'v', 'do', 'o')))
        lse = g.buffer(f'lse{r}', cfg.batch * H * T, 1, init={'kind': 'fill', 'value': 5.0})
        delta = g.buffer(f'delta{r}', cfg.batch * H * T, 1)
        dq, dk, dv = (g.buffer(f'd{n}{r}', N, d, 'bf16') for n in 'qkv')
        e.attention_bwd(f'b{r}', q, k, v, o, lse, do, delta, dq, dk, dv)
    ms, b = timed(g)
    fl = float(task_flops(b).sum())
    out['attention_bwd'] = {'tasks': len(b.tasks), 'ms': ms, 'achieved': fl / (ms * 1e-3) / 1e12, 'unit': 'TFLOP/s', 'peak': tfl, 'frac': fl / (ms * 1e-3) / 1e12 / tfl, 'bound': 'tensor',
                            'note': 'delta, dq and dkv tasks of one layer, dq / dkv after delta'}

    def mem(name, g, nbytes):
        ms, b = timed(g)
        gbs = nbytes / (ms * 1e-3) / 1e9
        out[name] = {'tasks': len(b.tasks), 'ms': ms, 'achieved': gbs, 'unit': 'GB/s', 'peak': hbm, 'frac': gbs / hbm, 'bound': 'hbm', 'algorithmic_bytes': nbytes}

    # ---- layernorm forward: x f32 -> out bf16 (+ mean, rstd), 4 copies of the [N, d] activation
    reps = 6
    e = emitter(); g = e.g
    gam, bet = g.buffer('gam', 1, d, init={'kind': 'fill', 'value': 1.0}), g.buffer('bet', 1, d)
    for r in range(reps):
        x = g.buffer(f'x{r}', N, d, init=sd(r + 1, 1.0))
        e.layernorm(f'ln{r}', x, gam, bet, g.buffer(f'h{r}', N, d, 'bf16'), g.buffer(f'mu{r}', N, 1), g.buffer(f'rs{r}', N, 1))
    mem('layernorm_fwd', g, reps * N * (d * 6 + 8))
    # ---- layernorm backward dx (acc = 1): x f32, dy bf16, dx f32 read + written
    e = emitter(); g = e.g
    e.params = {}
    g.buffer('w.p.g', 1, d, init={'kind': 'fill', 'value': 1.0})
    for r in range(reps):
        x, dy = g.buffer(f'x{r}', N, d, init=sd(r + 1, 1.0)), g.buffer(f'dy{r}', N, d, 'bf16', sd(r + 50, 1.0))
        mu, rs = g.buffer(f'mu{r}', N, 1), g.buffer(f'rs{r}', N, 1, init={'kind': 'fill', 'value': 1.0})
        dx = g.buffer(f'dx{r}', N, d)
        e._rowwise = {x, dy, dx}
        e.rows('layernorm_bwd_dx', f'lnb{r}', N, cfg.norm_rows, {'x': x, 'dy': dy, 'gamma': 'w.p.g', 'mean': mu, 'rstd': rs, 'dx': dx, 'd': d, 'acc': 1},
               [x, dy, 'w.p.g', dx], [dx], vec_r=[mu, rs])
    mem('layernorm_bwd_dx', g, reps * N * (d * 14 + 8))
    # ---- fused cross entropy over bf16 logits: one read + one write of [N, V] (the second read of a row comes from cache)
    e = emitter(); g = e.g
    logits, dlog = g.buffer('logits', N, V, 'bf16', sd(1, 1.0)), g.buffer('dlogits', N, V, 'bf16')
    tgt = g.buffer('tgt', N, 1, 'i32')
    e._rowwise = {logits}
    e.rows('softmax_ce_fused', 'ce', N, cfg.ce_rows, {'logits': logits, 'tgt': tgt, 'rowloss': g.buffer('rl', N, 1), 'lse': g.buffer('ls', N, 1), 'dlogits': dlog, 'V': V,
                                                       'ignore': -1, 'N': N, 'scale': 1.0}, [logits], [dlog], vec_r=[tgt], vec_w=['rl', 'ls'])
    mem('softmax_ce_fused', g, N * V * 4)
    # ---- AdamW over 64 M parameters: p, g, m, v read, p, m, v written
    e = emitter(); g = e.g
    n_par = 64 << 20
    for nm, init in (('p', sd(1, 0.02)), ('gr', sd(2, 0.01)), ('m', None), ('v', None)):
        g.buffer(nm, n_par // 4096, 4096, init=init)
    g.buffer('clip', 1, 2, init={'kind': 'fill', 'value': 1.0}); g.buffer('step', 1, 1, 'i32', {'kind': 'fill', 'value': 1})
    for i, (e0, e1) in enumerate(g.flat_chunks('p', cfg.flat_chunk)):
        rr = g.region_of('p', e0, e1)
        g.task('adamw', {'p': 'p', 'g': 'gr', 'm': 'm', 'v': 'v', 'gscale': 'clip', 'step': 'step', 'e0': e0, 'e1': e1, 'lr': 6e-4, 'b1': 0.9, 'b2': 0.999, 'eps': 1e-8, 'wd': 0.1},
               [('gr', *rr), 'clip', 'step'], [('p', *rr), ('m', *rr), ('v', *rr)], 1, f'adamw.{i}')
    mem('adamw', g, n_par * 28)
    # ---- residual add (f32 a + b -> out) and the f32 -> bf16 operand copy, over [N, F]-sized flats
    for name, op, outdt, per in (('residual_add', 'residual_add', 'f32', 12), ('round_bf16', 'round_bf16', 'bf16', 6)):
        e = emitter(); g = e.g
        for r in range(4):
            a = g.buffer(f'a{r}', N, F, init=sd(r + 1, 1.0))
            o = g.buffer(f'o{r}', N, F, outdt)
            if op == 'residual_add':
                bb = g.buffer(f'b{r}', N, F, init=sd(r + 9, 1.0))
                e.flat(op, [a, bb], [o], N * F, {'a': a, 'b': bb, 'out': o}, f'{op}{r}')
            else:
                e.flat(op, [a], [o], N * F, {'x': a, 'out': o}, f'{op}{r}')
        mem(name, g, 4 * N * F * per)
    # ---- column reductions at the step's granularity (64 columns x all rows per task): bias gradients (colsum of a bf16 [N, F]
    #      activation gradient) and the norm layers' dgamma / dbeta (x and dy bf16, mean and rstd per row)
    from kvm_b200.workloads.graph import Graph
    g = Graph('alone')
    reps = 3
    for r in range(reps):
        x = g.buffer(f'x{r}', N, F, 'bf16', sd(r + 1, 1.0))
        o = g.buffer(f'o{r}', 1, F)
        for c0 in range(0, F, cfg.col_chunk):
            g.task('colsum', {'x': x, 'out': o, 'R': N, 'c0': c0, 'c1': min(c0 + cfg.col_chunk, F), 'acc': 0})
    mem('colsum', g, reps * N * F * 2)
    g = Graph('alone')
    for r in range(reps):
        x, dy = g.buffer(f'x{r}', N, F, 'bf16', sd(r + 1, 1.0)), g.buffer(f'dy{r}', N, F, 'bf16', sd(r + 11, 1.0))
        mu, rs = g.buffer(f'mu{r}', 1, N, init=sd(r + 21, 1.0)), g.buffer(f'rs{r}', 1, N, init=sd(r + 31, 1.0))
        dg, db = g.buffer(f'dg{r}', 1, F), g.buffer(f'db{r}', 1, F)
        for c0 in range(0, F, cfg.col_chunk):
            g.task('norm_bwd_params', {'x': x, 'dy': dy, 'mean': mu, 'rstd': rs, 'dgamma': dg, 'dbeta': db, 'R': N, 'd': F, 'c0': c0, 'c1': min(c0 + cfg.col_chunk, F), 'acc': 0})
    mem('norm_bwd_params', g, reps * N * F * 4)
    return out


def run_small(device):
    """The two small configurations of the reference's benchmark list: the tiny GPT (2 layers, d 128, batch 8 x 64, f32, AdamW,
    20 steps unrolled in one launch) and eight MLPs of different widths trained side by side (batch 256, f32, SGD with momentum,
    10 steps in one launch), each on the ready-queue path and on the static-schedule path (per-worker task lists planned on the
    host: a dependent hop is one progress-word poll instead of a trip through the queue)."""
    from kvm_b200.executor import CFG_DYNAMIC, CFG_STATIC, Executor
    from kvm_b200.workloads.gpt import build_training, preset as gpt_preset
    from kvm_b200.workloads.mlp import build_mlps, params, preset as mlp_preset
    out = {}
    b = build_training(gpt_preset('gpt_tiny'), 20, stream_steps=80).to_bundle(check=False)
    c = mlp_preset('mlp8')
    bm = build_mlps(c, 10).to_bundle(check=False)
    for tag, flags in (('queue', CFG_DYNAMIC), ('static', CFG_STATIC)):
        with Executor(device=device, flags=flags) as ex:
            ex.load(b); ex.run()
            ms = min(ex.run().ms for _ in range(2))
            out.setdefault('gpt_tiny', {'tasks_per_step': len(b.tasks) // 20})[tag] = {
                'steps_per_s': 20 / (ms * 1e-3), 'us_per_step': ms * 1e3 / 20, 'loss_step0': float(ex.read_buffer('loss.0')[0, 0]), 'loss_step19': float(ex.read_buffer('loss.19')[0, 0])}
        with Executor(device=device, flags=flags) as ex:
            ex.load(bm); ex.run()
            ms = min(ex.run().ms for _ in range(2))
            out.setdefault('mlp8', {'tasks_per_step': len(bm.tasks) // 10, 'params': params(c), 'gflop_per_step': 6.0 * params(c) * c.batch / 1e9})[tag] = {'us_per_joint_step': ms * 1e3 / 10}
    return out


def run_355m(device, steps=3):
    """BASELINE configs[3], bf16 run: GPT-355M (24 layers, d 1024, 16 heads, FFN 4096, vocabulary 50304, T 1024), micro-batch 8, one
    persistent-kernel launch per step; a few steps, reported beside the headline with its own roofline fraction."""
    from kvm_b200.executor import Executor
    cfg, bundle = get_bundle('gpt_355m', 0, 1, 2 * steps + 6, {})
    with Executor(device=device) as ex:
        ex.load(bundle)
        ex.run_steps(2)
        res = ex.run_steps(steps)
        loss = float(ex.read_buffer('loss.0')[0, 0])
        tc = ex.tc_task_count()
    g, a = algorithmic_flops(cfg)
    pk, kind = peaks()
    peak = pk.get('bf16_tflops_sustained', PEAK_FALLBACK['bf16_tflops_sustained'])
    ms = res.ms / steps
    return {'workload': workload_name('gpt_355m', cfg), 'ms_per_step': ms, 'steps_per_s': 1e3 / ms, 'tasks': len(bundle.tasks), 'tc_tasks': tc, 'loss': loss,
            'roofline': {'bound': 'tensor', 'achieved': (g + a) / (ms * 1e-3) / 1e12, 'unit': 'TFLOP/s', 'peak': peak, 'frac': (g + a) / (ms * 1e-3) / 1e12 / peak,
                         'flops_per_launch': g + a, 'peak_source': f'{kind} bf16_tflops_sustained'}}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--gpus', type=int, default=1)
    ap.add_argument('--steps', type=int, default=10)
    ap.add_argument('--warmup', type=int, default=3)
    ap.add_argument('--impl', default='ours', choices=['ours', 'reference'])
    ap.add_argument('--model', default='gpt_162m')
    ap.add_argument('--decode-model', default='qwen3_8b')
    ap.add_argument('--decode-tokens', type=int, default=128, help='tokens of the decode measurement appended to the line (0 = skip)')
    ap.add_argument('--extras', default='decode,alone,small,355m', help='objects appended to the line at one GPU: decode, alone (kernels_alone), small (small_models), 355m; empty for none (profiling runs)')
    ap.add_argument('--cpu-seconds', type=float, default=15.0, help='length of the CPU-oracle sample behind cpu_baseline (0 = skip)')
    ap.add_argument('--cpu-step-limit', type=float, default=240.0, help='--impl reference: time limit of the one real CPU step')
    args = ap.parse_args()
    rank, world, local_rank = int(os.environ.get('RANK', 0)), int(os.environ.get('WORLD_SIZE', 1)), int(os.environ.get('LOCAL_RANK', 0))
    args.warmup = max(args.warmup, 3) if args.impl == 'ours' else args.warmup
    if args.impl == 'reference':
        run_reference(args, rank, world)
    elif world > 1:
        run_dp(args, rank, world, local_rank)
    else:
        run_ours(args, rank, world, local_rank)


if __name__ == '__main__':
    main()
