"""Data-parallel training step: backward bundle -> gradient all-reduce -> optimizer bundle, one process per GPU.

The semantics are the reference planner's (`runtime/partition.py:1301-1386`, DPPlanner): rank r trains on microbatch r of each
group of P, every gradient is averaged over the P ranks before its first reader (the gradient-norm partials), clip and AdamW
then run redundantly on identical values, so the replicas stay equal and the result equals gradient accumulation over P
microbatches.  The reference builds the exchange from peer-store tasks inside its kernel.  Two forms here: `DataParallelStep`, one NCCL
all-reduce (supplied by the caller, e.g. torch.distributed) over a single arena that holds every gradient buffer, between two
launches of the persistent kernel; and `DataParallelStepFused`, ONE launch per step and rank in which the all-reduce is tasks of
the graph (peer stores into the other ranks' memory over NVLink, flag words, bounded waits: `_Emit.dp_exchange`), running while
the backward still has work.
"""
from __future__ import annotations

import numpy as np

from .executor import Executor
from .workloads.gpt import GPTConfig, build_training, dp_exchange_layout


def grad_arena_layout(bundle):
    """{buffer index: (offset_elems, n_elems)} of the f32 gradient buffers ('g.*') inside one contiguous arena, 64-element
    (256-byte) aligned so vector accesses and TMA stay legal; and the arena length."""
    lay, off = {}, 0
    for b in bundle.buffers:
        if b['name'].startswith('g.') and b['dtype'] == 0:
            n = b['rows'] * b['cols']
            lay[b['index']] = (off, n)
            off += -(-n // 64) * 64
    return lay, off


class DataParallelStep:
    """Two executor handles over one buffer table: `bwd` (data window, forward, backward) and `opt` (clip, AdamW, publishes)."""

    def __init__(self, cfg: GPTConfig, rank: int, world: int, device: int, arena_ptr: int, stream_steps: int, bundles=None, **exec_kw):
        if bundles is None:
            g = build_training(cfg, 1, rank=rank, world=world, stream_steps=stream_steps)
            bundles = g.to_bundles_split(g.split_at)
        self.b_bwd, self.b_opt = bundles
        self.layout, self.arena_elems = grad_arena_layout(self.b_bwd)
        self.bwd = Executor(device=device, **exec_kw)
        for spec in self.b_bwd.buffers:
            if spec['index'] in self.layout:      # gradients live in the caller's arena so one collective covers them all
                self.bwd.bind_buffer(arena_ptr + 4 * self.layout[spec['index']][0], spec['rows'], spec['cols'], 0, name=spec['name'])
            else:
                self.bwd.add_bundle_buffer(self.b_bwd, spec)
        self.bwd.submit(self.b_bwd.tasks, self.b_bwd.succ, self.b_bwd.args)
        self.bwd.bundle = self.b_bwd
        self.opt = Executor(device=device, **exec_kw)
        for spec in self.b_opt.buffers:
            self.opt.bind_buffer(self.bwd.buffer_ptr(spec['index']), spec['rows'], spec['cols'], spec['dtype'], name=spec['name'])
        self.opt.submit(self.b_opt.tasks, self.b_opt.succ, self.b_opt.args)
        self.opt.bundle = self.b_opt

    def step(self, all_reduce_mean):
        """all_reduce_mean(): averages the arena over the ranks in place and returns when the result is visible to the device."""
        r1 = self.bwd.run()
        all_reduce_mean()
        r2 = self.opt.run()
        return r1, r2

    def close(self):
        self.opt.close()
        self.bwd.close()


class DataParallelStepFused:
    """One executor per rank, one launch per step: the gradient all-reduce is part of the graph.  `exchange_handles(mine: dict) ->
    list[dict]` is the caller's all-gather of small Python objects over the ranks; every rank exports its arena, inbox and flag
    buffers (kvm_ipc_export), maps the peers' (kvm_ipc_open) and binds them as the graph's `dp.peer{p}.*` buffers; the gradient
    buffers `g.*` are bound to slices of the rank's own arena, so a peer's store into the arena is a store into the gradient."""
    OWN = ('dp.arena', 'dp.inbox', 'dp.flag', 'dp.gflag')

    def __init__(self, cfg: GPTConfig, rank: int, world: int, device: int, stream_steps: int, exchange_handles, bundle=None, **exec_kw):
        self.cfg, self.rank, self.world = cfg, rank, world
        self.bundle = b = bundle or build_training(cfg, 1, rank=rank, world=world, stream_steps=stream_steps, dp_fused=True).to_bundle(check=False)
        arena, self.arena_elems, _, _, _ = dp_exchange_layout(cfg, world)
        self.ex = ex = Executor(device=device, **exec_kw)
        self._mapped, peers = [], None
        for spec in b.buffers:
            name = spec['name']
            if name.startswith('dp.peer'):
                if peers is None:
                    peers = exchange_handles({n.split('.')[1]: ex.ipc_export(n) for n in self.OWN})
                p, what = int(name.split('.')[1][4:]), name.split('.')[2]
                ptr = ex.ipc_open(peers[p][what])
                self._mapped.append(ptr)
                ex.bind_buffer(ptr, spec['rows'], spec['cols'], spec['dtype'], name=name)
            elif name.startswith('g.') and name[2:] in arena:
                ex.bind_buffer(ex.buffer_ptr('dp.arena') + 4 * arena[name[2:]], spec['rows'], spec['cols'], 0, name=name)
            else:
                ex.add_bundle_buffer(b, spec)
        ex.submit(b.tasks, b.succ, b.args)
        ex.bundle = b
        self.bwd = self.opt = ex          # the names the two-launch form uses for its handles

    def step(self):
        return self.ex.run()

    def close(self):
        for ptr in self._mapped:
            self.ex.L.kvm_ipc_close(self.ex._h, ptr)
        self._mapped = []
        self.ex.close()
