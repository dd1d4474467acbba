"""Data parallelism on CPU ranks (gloo, world size 2) with the oracle as the engine: the per-rank token split, the
backward / all-reduce / optimizer split of the step, and the reference planner's contract that the replicas end bit-identical
and equal to gradient accumulation over the two microbatches (runtime/partition.py:1302-1311 of the reference)."""
import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from kvm_b200.dp import grad_arena_layout
from kvm_b200.workloads.gpt import build_training, preset
from oracle.vm_np import VM


def _run_rank_halves(rank, world, reduce_fn):
    cfg = preset('gpt_micro')
    g = build_training(cfg, 1, rank=rank, world=world, stream_steps=2)
    b_bwd, b_opt = g.to_bundles_split(g.split_at)
    lay, n = grad_arena_layout(b_bwd)
    vm = VM(b_bwd)
    for step in range(2):
        vm.run()
        arena = np.zeros(n, np.float32)
        for idx, (off, cnt) in lay.items():
            arena[off:off + cnt] = vm.bufs[idx].a.reshape(-1)
        arena = reduce_fn(arena)
        for idx, (off, cnt) in lay.items():
            vm.bufs[idx].a.reshape(-1)[:] = arena[off:off + cnt]
        vo = VM(b_opt, buffers=vm.bufs)
        vo.run()
        vm = VM(b_bwd, buffers=vo.bufs)
    names = [s['name'] for s in b_bwd.buffers if s['name'].startswith('w.')]
    return {nme: vm.buffer(nme).a.copy() for nme in names}


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR='127.0.0.1', MASTER_PORT=str(port))
    dist.init_process_group('gloo', rank=rank, world_size=world)

    def reduce_fn(arena):
        t = torch.from_numpy(arena)
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        return (t * (1.0 / world)).numpy()

    w = _run_rank_halves(rank, world, reduce_fn)
    q.put((rank, {k: v.tobytes() for k, v in w.items()}))
    dist.barrier()
    dist.destroy_process_group()


def test_two_ranks_equal_gradient_accumulation():
    with socket.socket() as s:
        s.bind(('127.0.0.1', 0))
        port = s.getsockname()[1]
    ctx = mp.get_context('spawn')
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = dict(q.get(timeout=300) for _ in range(2))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert got[0].keys() == got[1].keys()
    for k in got[0]:
        assert got[0][k] == got[1][k], f'replicas diverged on {k}'
    # single-process reference: both microbatches, gradients averaged, one optimizer step per step
    cfg = preset('gpt_micro')
    gs = [build_training(cfg, 1, rank=r, world=2, stream_steps=2) for r in range(2)]
    halves = [g.to_bundles_split(g.split_at) for g in gs]
    lay, n = grad_arena_layout(halves[0][0])
    vms = [VM(h[0]) for h in halves]
    for step in range(2):
        for vm in vms:
            vm.run()
        for idx in lay:
            avg = (vms[0].bufs[idx].a + vms[1].bufs[idx].a) * np.float32(0.5)
            for vm in vms:
                vm.bufs[idx].a[:] = avg
        nxt = []
        for vm, h in zip(vms, halves):
            vo = VM(h[1], buffers=vm.bufs)
            vo.run()
            nxt.append(VM(h[0], buffers=vo.bufs))
        vms = nxt
    for k in got[0]:
        assert vms[0].buffer(k).a.tobytes() == got[0][k], f'{k} differs from gradient accumulation'
    # and the step really moved the weights
    fresh = VM(halves[0][0])
    assert any(fresh.buffer(k).a.tobytes() != got[0][k] for k in got[0])


import pytest


@pytest.mark.parametrize('world', [2, 4])
def test_fused_exchange_graphs_equal_gradient_accumulation(world):
    """The one-launch form: the all-reduce is tasks of each rank's graph (peer_put_signal / peer_wait_sum / peer_wait).  The oracle
    VMs of the ranks run as threads; a rank's `dp.peer{p}.*` buffers are the other rank's arrays and every gradient buffer is a view
    into the rank's arena (what the GPU runner sets up with CUDA IPC and kvm_bind_buffer).  With 2 or 4 ranks the result is
    bit-identical to summing the microbatch gradients in rank order and scaling by 1 / world (the 1 / world folded into the loss
    gradient is an exact scaling by a power of two)."""
    import threading
    from kvm_b200.workloads.gpt import dp_exchange_layout
    from oracle.ops_np import Buf
    cfg = preset('gpt_micro')
    bundles = [build_training(cfg, 1, rank=r, world=world, stream_steps=2, dp_fused=True).to_bundle() for r in range(world)]
    arena, n_arena, chunks, width, owned = dp_exchange_layout(cfg, world)
    index = lambda b, name: next(i for i, spec in enumerate(b.buffers) if spec['name'] == name)
    vms = [VM(b) for b in bundles]
    for vm, b in zip(vms, bundles):
        flat = vm.buffer('dp.arena').a.reshape(-1)
        for name, off in arena.items():
            i = index(b, 'g.' + name)
            spec = b.buffers[i]
            vm.bufs[i] = Buf(flat[off:off + spec['rows'] * spec['cols']].reshape(spec['rows'], spec['cols']), 0)
    for r in range(world):
        for p in range(world):
            if p != r:
                for what in ('arena', 'inbox', 'flag', 'gflag'):
                    vms[r].bufs[index(bundles[r], f'dp.peer{p}.{what}')] = vms[p].buffer(f'dp.{what}')
    for step in range(2):
        errs = []

        def run(vm):
            try:
                vm.run()
            except Exception as e:
                errs.append(e)
        th = [threading.Thread(target=run, args=(vm,)) for vm in vms]
        for t in th:
            t.start()
        for t in th:
            t.join(timeout=300)
        assert not errs, errs
        vms = [VM(b, buffers=vm.bufs) for b, vm in zip(bundles, vms)]
    wnames = [s['name'] for s in bundles[0].buffers if s['name'].startswith('w.')]
    for k in wnames:
        for r in range(1, world):
            assert np.array_equal(vms[0].buffer(k).a, vms[r].buffer(k).a), f'replicas diverged on {k}'
    # reference: the two-launch form with the mean taken on the host, partials added in rank order
    gs = [build_training(cfg, 1, rank=r, world=world, stream_steps=2) for r in range(world)]
    halves = [g.to_bundles_split(g.split_at) for g in gs]
    lay, n = grad_arena_layout(halves[0][0])
    ref = [VM(h[0]) for h in halves]
    for step in range(2):
        for vm in ref:
            vm.run()
        for idx in lay:
            acc = ref[0].bufs[idx].a.copy()
            for r in range(1, world):
                acc = (acc + ref[r].bufs[idx].a).astype(np.float32)
            avg = acc * np.float32(1.0 / world)
            for vm in ref:
                vm.bufs[idx].a[:] = avg
        nxt = []
        for vm, h in zip(ref, halves):
            vo = VM(h[1], buffers=vm.bufs)
            vo.run()
            nxt.append(VM(h[0], buffers=vo.bufs))
        ref = nxt
    for k in wnames:
        assert np.array_equal(vms[0].buffer(k).a, ref[0].buffer(k).a), f'{k} differs from gradient accumulation'
