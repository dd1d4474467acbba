"""Tensor-parallel greedy decode, one process per GPU: the token's graph is cut at the two partial-sum points of every layer
(after the attention-output projection and after the down projection) into 2 * layers + 1 segments; each segment is one
launch of the persistent kernel, and between two segments the `[1, hidden]` partial is summed over the ranks by the caller's
collective (NCCL through torch.distributed in bench.py).  The LM head is sharded by vocabulary: every rank proposes the best
token of its slice and the best proposal wins (lowest index on ties, as `argmax` does).

This is what the reference plans with its tensor-parallel partitioner and in-kernel comm ops (`runtime/partition.py`,
include/mvm_ops_comm.def).  Two forms: `TensorParallelDecode` (the exchange is a library collective between launches) and
`TensorParallelDecodeFused` (ONE launch per token and rank: the sums are tasks that store the partial into the peers' inboxes
over NVLink, release a flag word and wait, bounded, for the peers' flags; extension ops 302 / 303).
"""
from __future__ import annotations

import numpy as np

from .executor import Executor
from .workloads.decode import DecodeConfig, build_decode_tp


def pick_token(proposals):
    """proposals: iterable of (best logit, global index) per rank -> the global greedy token (lowest index among equal logits)."""
    best = None
    for val, idx in proposals:
        if best is None or val > best[0] or (val == best[0] and idx < best[1]):
            best = (val, idx)
    return int(best[1])


class TensorParallelDecode:
    """Executor handles of one rank: handle 0 owns the buffers (the exchanged partials, the logits slice and the token are
    bound to caller memory so collectives can run on them), the others share them."""

    def __init__(self, cfg: DecodeConfig, rank: int, world: int, device: int, bind: dict, exact: bool = False, **exec_kw):
        """bind: {buffer name: device pointer} for every exchanged buffer, 'u0.logits' and 'u0.tok' (float32 / int32 storage)."""
        self.cfg, self.rank, self.world = cfg, rank, world
        g, cuts, self.exchanges = build_decode_tp(cfg, rank, world, exact)
        self.bundles = g.to_bundles_multi(cuts)
        first = self.bundles[0]
        self.handles = []
        ex0 = Executor(device=device, **exec_kw)
        for spec in first.buffers:
            if spec['name'] in bind:
                ex0.bind_buffer(bind[spec['name']], spec['rows'], spec['cols'], spec['dtype'], name=spec['name'])
            else:
                ex0.add_bundle_buffer(first, spec)
        ex0.submit(first.tasks, first.succ, first.args)
        ex0.bundle = first
        self.handles.append(ex0)
        for b in self.bundles[1:]:
            ex = Executor(device=device, **exec_kw)
            for spec in b.buffers:
                ex.bind_buffer(ex0.buffer_ptr(spec['index']), spec['rows'], spec['cols'], spec['dtype'], name=spec['name'])
            ex.submit(b.tasks, b.succ, b.args)
            ex.bundle = b
            self.handles.append(ex)

    def token(self, all_reduce_sum, choose):
        """One decode step. all_reduce_sum(name): sums that bound buffer over the ranks in place, visible to the device on return.
        choose(): reduces the ranks' logits slices to the next token and writes it to the bound 'u0.tok' on every rank."""
        ms = 0.0
        for ex, name in zip(self.handles, self.exchanges):
            ms += ex.run().ms
            if name is not None:
                all_reduce_sum(name)
        choose()
        return ms

    def use_stream(self, cuda_stream: int):
        """Put every handle on the caller's stream (needs the handles created with flags=CFG_CHAIN): token_async then needs no host
        synchronisation between segments."""
        for ex in self.handles:
            ex.set_stream(cuda_stream)

    def token_async(self, all_reduce_sum, choose):
        """One decode step queued on the shared stream: launches and collectives follow each other in stream order; `choose` ends
        with whatever synchronisation the token read-back needs."""
        for ex, name in zip(self.handles, self.exchanges):
            ex.start()
            if name is not None:
                all_reduce_sum(name)
        choose()

    def finish(self):
        """Collect the last results of every handle (raises on a recorded device error); returns their kernel times in ms."""
        return [ex.finish().ms for ex in self.handles]

    def close(self):
        for ex in reversed(self.handles):
            ex.close()


class TensorParallelDecodeFused:
    """One executor per rank, one launch per token: the partial sums over the ranks are tasks of the graph (peer_put_signal /
    peer_wait_sum).  `exchange_handles(handles: dict) -> list[dict]` is the caller's all-gather of small Python objects over the
    ranks (torch.distributed.all_gather_object in bench.py): every rank exports its inbox and flag buffers, maps the peers' and
    binds them as the graph's `tp.peer{p}.*` buffers.  Only the token choice (one proposal per rank) stays with the caller."""

    def __init__(self, cfg: DecodeConfig, rank: int, world: int, device: int, bind: dict, exchange_handles, exact: bool = False, **exec_kw):
        self.cfg, self.rank, self.world = cfg, rank, world
        g, _, _ = build_decode_tp(cfg, rank, world, exact, fused=True)
        self.bundle = b = g.to_bundle(check=False)
        self.ex = ex = Executor(device=device, **exec_kw)
        self._mapped = []
        peers = None
        for spec in b.buffers:
            name = spec['name']
            if name.startswith('tp.peer'):
                if peers is None:            # this rank's inbox and flag words exist by now (they are the first buffers of the graph)
                    mine = {'inbox': ex.ipc_export('tp.inbox'), 'flag': ex.ipc_export('tp.flag')}
                    peers = exchange_handles(mine)
                p, what = int(name.split('.')[1][4:]), name.split('.')[2]
                ptr = ex.ipc_open(peers[p][what])
                self._mapped.append(ptr)
                ex.bind_buffer(ptr, spec['rows'], spec['cols'], spec['dtype'], name=name)
            elif name in bind:
                ex.bind_buffer(bind[name], spec['rows'], spec['cols'], spec['dtype'], name=name)
            else:
                ex.add_bundle_buffer(b, spec)
        ex.submit(b.tasks, b.succ, b.args)
        ex.bundle = b
        self.handles = [ex]

    def token(self, choose):
        """One decode step: one launch, then the caller's token choice over the ranks' logits slices."""
        ms = self.ex.run().ms
        choose()
        return ms

    def use_stream(self, cuda_stream: int):
        self.ex.set_stream(cuda_stream)

    def token_async(self, choose):
        self.ex.start()
        choose()

    def finish(self):
        return [self.ex.finish().ms]

    def close(self):
        for ptr in self._mapped:
            self.ex.L.kvm_ipc_close(self.ex._h, ptr)
        self._mapped = []
        self.ex.close()
