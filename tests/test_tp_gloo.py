"""Tensor-parallel decode on CPU ranks (gloo, world size 2) with the oracle as the engine: the sharding of the one-token graph
(heads / FFN columns / vocabulary), the two partial-sum exchanges per layer and the token choice over the vocabulary slices
must reproduce the unsharded graph's greedy tokens and hidden state."""
import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from kvm_b200.tp import pick_token
from kvm_b200.workloads.decode import build_decode, build_decode_tp, preset
from oracle.vm_np import VM

CFG = dict(init_std=0.08)      # large enough logit gaps that the two summation orders agree on every token
NTOK = 3


def _reference_tokens():
    b = build_decode(preset('decode_tiny', **CFG)).to_bundle()
    vm, toks = VM(b), []
    for _ in range(NTOK):
        vm.run()
        toks.append(int(vm.buffer('u0.tok').a[0, 0]))
        vm = VM(b, buffers=vm.bufs)
    return toks, vm.buffer('u0.logits').a.copy()


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR='127.0.0.1', MASTER_PORT=str(port))
    dist.init_process_group('gloo', rank=rank, world_size=world)
    c = preset('decode_tiny', **CFG)
    g, cuts, exchanges = build_decode_tp(c, rank, world, exact=True)
    bundles = g.to_bundles_multi(cuts)
    bufs, toks = None, []
    Vl = c.vocab // world
    for _ in range(NTOK):
        for b, name in zip(bundles, exchanges):
            vm = VM(b, buffers=bufs)
            vm.run()
            bufs = vm.bufs
            if name is not None:
                t = torch.from_numpy(vm.buffer(name).a)
                dist.all_reduce(t, op=dist.ReduceOp.SUM)
        lg = vm.buffer('u0.logits').a[0]
        mine = torch.tensor([float(lg.max()), float(rank * Vl + int(lg.argmax()))], dtype=torch.float64)
        allp = [torch.zeros(2, dtype=torch.float64) for _ in range(world)]
        dist.all_gather(allp, mine)
        tok = pick_token((float(p[0]), int(p[1])) for p in allp)
        vm.buffer('u0.tok').a[0, 0] = tok
        toks.append(tok)
    q.put((rank, toks, vm.buffer('u0.logits').a.tobytes()))
    dist.barrier()
    dist.destroy_process_group()


def test_two_ranks_reproduce_the_unsharded_tokens():
    ref_toks, ref_logits = _reference_tokens()
    with socket.socket() as s:
        s.bind(('127.0.0.1', 0))
        port = s.getsockname()[1]
    ctx = mp.get_context('spawn')
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = sorted(q.get(timeout=300) for _ in range(2))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert got[0][1] == got[1][1] == ref_toks, (got[0][1], got[1][1], ref_toks)
    logits = np.concatenate([np.frombuffer(r[2], np.float32) for r in got])
    assert np.allclose(logits, ref_logits.ravel(), rtol=2e-3, atol=2e-3)      # partial sums in another order, bf16-rounded activations


def test_pick_token_prefers_the_lowest_index_on_ties():
    assert pick_token([(1.0, 7), (2.0, 9), (2.0, 3)]) == 3


def test_fused_exchange_graphs_reproduce_the_unsharded_tokens():
    """The one-launch form: each rank's whole token is one graph whose partial sums are peer_put_signal / peer_wait_sum tasks.
    Two oracle VMs run as threads of this process; a rank's `tp.peer{p}.*` buffers are the other rank's `tp.inbox` / `tp.flag`
    arrays (what the GPU runner maps over CUDA IPC), so a put lands in the peer's memory and its wait really waits for it."""
    import threading
    ref_toks, ref_logits = _reference_tokens()
    c = preset('decode_tiny', **CFG)
    world, Vl = 2, c.vocab // 2
    bundles = [build_decode_tp(c, r, world, exact=True, fused=True)[0].to_bundle() for r in range(world)]
    assert [s['name'] for s in bundles[0].buffers[:4]] == ['tp.inbox', 'tp.flag', 'tp.peer1.inbox', 'tp.peer1.flag']
    vms = [VM(b) for b in bundles]
    index = lambda b, name: next(i for i, spec in enumerate(b.buffers) if spec['name'] == name)
    for r in range(world):                                  # bind the peer views: the same Buf objects, hence the same arrays
        for p in range(world):
            if p != r:
                vms[r].bufs[index(bundles[r], f'tp.peer{p}.inbox')] = vms[p].buffer('tp.inbox')
                vms[r].bufs[index(bundles[r], f'tp.peer{p}.flag')] = vms[p].buffer('tp.flag')
    toks = []
    for _ in range(NTOK):
        errs = []

        def run(vm):
            try:
                vm.run()
            except Exception as e:      # surfaces in the asserting thread
                errs.append(e)
        th = [threading.Thread(target=run, args=(vm,)) for vm in vms]
        for t in th:
            t.start()
        for t in th:
            t.join(timeout=120)
        assert not errs, errs
        props = []
        for r, vm in enumerate(vms):
            lg = vm.buffer('u0.logits').a[0]
            props.append((float(lg.max()), r * Vl + int(lg.argmax())))
        tok = pick_token(props)
        toks.append(tok)
        vms = [VM(b, buffers=vm.bufs) for b, vm in zip(bundles, vms)]
        for vm in vms:
            vm.buffer('u0.tok').a[0, 0] = tok
    assert toks == ref_toks, (toks, ref_toks)
    logits = np.concatenate([vm.buffer('u0.logits').a.ravel() for vm in vms])
    assert np.allclose(logits, ref_logits.ravel(), rtol=2e-3, atol=2e-3)
    # the replicas of the summed hidden state are bit-equal: every rank adds the partials in rank order
    last = f'u0.l{c.layers - 1}.x2'
    assert np.array_equal(vms[0].buffer(last).a, vms[1].buffer(last).a)
