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
