"""The multi-GPU runners on ONE GPU: two ranks of `TensorParallelDecode` and of `DataParallelStep` live in one process on one
device and the collective between their launches is a host-side sum (the reference tests its distributed path the same way:
two executors in one process on one GPU, DISTRIBUTED.md:13).  What runs on the device is exactly what `bench.py --gpus N` runs
per rank: the sharded graphs, buffers bound to caller memory (kvm_bind_buffer), one handle per segment.  The ranks' launches are
sequential here, none waits for another.

  tensor parallel   greedy tokens of the 2-way sharded decode == tokens of the unsharded graph on the GPU == the oracle's
  data parallel     two ranks on their own microbatches, gradients averaged: replicas bit-identical, weights equal to the oracle's
                    gradient accumulation over the two microbatches (runtime/partition.py:1302-1311 of the reference)
"""
import numpy as np
import pytest

from tests.parity import rel_err

pytestmark = pytest.mark.gpu


def test_two_tensor_parallel_ranks_reproduce_the_unsharded_tokens(kvm_lib):
    import torch
    from kvm_b200.executor import Executor
    from kvm_b200.tp import TensorParallelDecode, pick_token
    from kvm_b200.workloads.decode import build_decode, preset
    from oracle.vm_np import VM
    cfg = preset('decode_tiny', init_std=0.08)
    ntok, world = 6, 2
    full = build_decode(cfg).to_bundle()
    vm, ref = VM(full), []
    for _ in range(ntok):
        vm.run()
        ref.append(int(vm.buffer('u0.tok').a[0, 0]))
        vm = VM(full, buffers=vm.bufs)
    with Executor() as ex:
        ex.load(full)
        single = []
        for _ in range(ntok):
            ex.run()
            single.append(int(ex.read_buffer('u0.tok')[0, 0]))
    assert single == ref

    names = [f'u0.l{l}.{n}' for l in range(cfg.layers) for n in ('x1', 'x2')]
    ranks, mem = [], []
    for r in range(world):
        m = {n: torch.zeros(1, cfg.hidden, dtype=torch.float32, device='cuda') for n in names}
        m['u0.logits'] = torch.zeros(1, cfg.vocab // world, dtype=torch.float32, device='cuda')
        m['u0.tok'] = torch.full((1, 1), 3 % cfg.vocab, dtype=torch.int32, device='cuda')
        torch.cuda.synchronize()
        mem.append(m)
        ranks.append(TensorParallelDecode(cfg, r, world, 0, {n: t.data_ptr() for n, t in m.items()}, exact=True))
    got = []
    for _ in range(ntok):
        for seg, name in enumerate(ranks[0].exchanges):
            for tpd in ranks:
                res = tpd.handles[seg].run()
                assert res.done == len(tpd.bundles[seg].tasks)
            if name is not None:                      # the all-reduce: sum of the ranks' partials, back into every rank's buffer
                total = mem[0][name] + mem[1][name]
                for m in mem:
                    m[name].copy_(total)
                torch.cuda.synchronize()
        props = []
        for r, m in enumerate(mem):
            val, idx = m['u0.logits'].max(dim=1)
            props.append((float(val.item()), int(idx.item()) + r * (cfg.vocab // world)))
        tok = pick_token(props)
        for m in mem:
            m['u0.tok'].fill_(tok)
        torch.cuda.synchronize()
        got.append(tok)
    for tpd in ranks:
        tpd.close()
    assert got == ref, (got, ref)


def test_two_data_parallel_ranks_equal_gradient_accumulation(kvm_lib):
    import torch
    from kvm_b200.dp import DataParallelStep, grad_arena_layout
    from kvm_b200.workloads.gpt import build_training, preset
    from oracle.vm_np import VM
    cfg, world, steps = preset('gpt_micro'), 2, 2
    graphs = [build_training(cfg, 1, rank=r, world=world, stream_steps=steps) for r in range(world)]
    halves = [g.to_bundles_split(g.split_at) for g in graphs]
    lay, n = grad_arena_layout(halves[0][0])
    arenas = [torch.zeros(n, dtype=torch.float32, device='cuda') for _ in range(world)]
    torch.cuda.synchronize()
    dps = [DataParallelStep(cfg, r, world, 0, arenas[r].data_ptr(), steps, bundles=halves[r]) for r in range(world)]
    for _ in range(steps):
        for dp in dps:
            assert dp.bwd.run().done == len(dp.b_bwd.tasks)
        mean = (arenas[0] + arenas[1]) * 0.5          # what ncclAllReduce(AVG) leaves on every rank
        for a in arenas:
            a.copy_(mean)
        torch.cuda.synchronize()
        for dp in dps:
            assert dp.opt.run().done == len(dp.b_opt.tasks)
    # the oracle: both microbatches, gradients averaged, one optimizer step per step
    vms = [VM(h[0]) for h in halves]
    for _ in range(steps):
        for vm in vms:
            vm.run()
        for idx in lay:
            avg = (vms[0].bufs[idx].a + vms[1].bufs[idx].a) * np.float32(0.5)
            for vm in vms:
                vm.bufs[idx].a[:] = avg
        nxt = []
        for vm, h in zip(vms, halves):
            vo = VM(h[1], buffers=vm.bufs).run()
            nxt.append(VM(h[0], buffers=vo.bufs))
        vms = nxt
    names = [s['name'] for s in halves[0][0].buffers if s['name'].startswith('w.')]
    moved = False
    for nme in names:
        w0, w1 = dps[0].bwd.read_buffer(nme), dps[1].bwd.read_buffer(nme)
        assert np.array_equal(w0.view(np.uint32), w1.view(np.uint32)), f'replicas diverged on {nme}'
        if 'attn.k.b' not in nme:
            assert rel_err(w0, vms[0].buffer(nme).a) <= 2e-5, nme
        moved |= not np.array_equal(w0, VM(halves[0][0]).buffer(nme).a)
    assert moved
    for dp in dps:
        dp.close()


# ---- the exchange ops of the one-launch tensor-parallel form (peer_put_signal 302, peer_wait_sum 303) on one GPU ------------------------
# No second kernel runs here (two kernels that wait for one another must not share a GPU): the "peer" is host code that fills this
# rank's inbox and flag word before the launch, or never does.
def _exchange_graph(n=4096, seq0=40):
    from kvm_b200.workloads.graph import Graph
    rng = np.random.default_rng(5)
    g = Graph('xchg')
    g.data('partial', rng.standard_normal((1, n)).astype(np.float32))
    g.data('res', rng.standard_normal((1, n)).astype(np.float32))
    g.buffer('inbox', 2 * 2, n), g.buffer('flag', 1, 2 * 2, 'i32')
    g.buffer('peer.inbox', 2 * 2, n), g.buffer('peer.flag', 1, 2 * 2, 'i32')      # stand-ins for the peer's memory
    g.data('seq', np.array([[seq0]], np.int32), 'i32')
    g.buffer('out', 1, n)
    site, rank, world = 1, 0, 2
    row0 = site * world
    g.task('peer_put_signal', {'src': 'partial', 'dst': 'peer.inbox', 'src_off': 0, 'dst_off': (row0 + rank) * n, 'n': n, 'flag': 'peer.flag', 'var': row0 + rank,
                               'ver': 1, 'seq': 'seq', 'stride': 1}, ['partial', 'seq'], ['peer.inbox', 'peer.flag'])
    g.task('peer_wait_sum', {'partial': 'partial', 'inbox': 'inbox', 'flag': 'flag', 'out': 'out', 'res': 'res', 'n': n, 'row0': row0, 'rank': rank, 'world': world,
                             'ver': 1, 'seq': 'seq', 'stride': 1, 'p_off': 0, 'o_off': 0}, ['partial', 'seq', 'inbox', 'flag', 'res'], ['out'])
    return g.to_bundle(), n, row0, seq0


@pytest.mark.parametrize('flags', ['static', 'queue'])
def test_exchange_ops_deliver_and_sum_in_rank_order(kvm_lib, flags):
    from kvm_b200.executor import CFG_DYNAMIC, CFG_STATIC, Executor
    from oracle.vm_np import VM
    b, n, row0, seq0 = _exchange_graph()
    theirs = np.random.default_rng(6).standard_normal((1, n)).astype(np.float32)
    vm = VM(b)
    vm.buffer('inbox').a[row0 + 1] = theirs[0]
    vm.buffer('flag').a[0, row0 + 1] = seq0 + 1
    vm.run()
    with Executor(flags=CFG_STATIC if flags == 'static' else CFG_DYNAMIC) as ex:
        ex.load(b)
        ex.write_buffer('inbox', theirs, offset_elems=(row0 + 1) * n)                  # what the peer's put would have stored ...
        ex.write_buffer('flag', np.array([seq0 + 1], np.int32), offset_elems=row0 + 1)    # ... and released
        res = ex.run()
        assert res.status == 0 and res.done == 2
        assert np.array_equal(ex.read_buffer('out'), vm.buffer('out').a)              # same order of additions: bit-equal
        assert np.array_equal(ex.read_buffer('peer.inbox'), vm.buffer('peer.inbox').a)
        assert ex.read_buffer('peer.flag').tolist() == vm.buffer('peer.flag').a.tolist() and ex.read_buffer('peer.flag')[0, row0] == seq0 + 1


def test_exchange_wait_runs_out_when_the_peer_never_signals(kvm_lib):
    """Failure detection without a fault: nothing sets the flag, the bounded wait ends after the launch timeout, the launch returns
    KVM_ERR_TIMEOUT for that task and the handle stays usable."""
    from kvm_b200 import abi
    from kvm_b200.executor import Executor
    b, n, row0, seq0 = _exchange_graph()
    with Executor(timeout_ms=300) as ex:
        ex.load(b)
        res = ex.run(check=False)
        assert abi.err_name(res.status) == 'TIMEOUT' and res.err_task == 1, (res.status, res.err_task)
        assert ex.read_buffer('peer.flag')[0, row0] == seq0 + 1                        # the put itself was delivered
        ex.write_buffer('flag', np.array([seq0 + 1], np.int32), offset_elems=row0 + 1)    # the peer arrives after all
        res = ex.run(check=False)
        assert res.status == 0 and res.done == 2
