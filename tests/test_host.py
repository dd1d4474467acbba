"""Host-side logic without a GPU: op registry, bundle compiler / validator, graph builder dataflow, the C ABI's symbols."""
import json
import re
from pathlib import Path

import numpy as np
import pytest

from kvm_b200 import abi
from kvm_b200.bundle import Bundle, CompileError, compile_spec, load_bundle, validate
from kvm_b200.workloads.gpt import build_training, preset, token_stream
from kvm_b200.workloads.graph import Graph
from oracle.vm_np import VM

ROOT = Path(__file__).resolve().parents[1]


def test_registry_ids_and_arities():
    ops = abi.load_ops()
    assert ops['noop'].id == 0 and ops['matmul_tile'].id == 34 and ops['matmul_mma_bf16'].id == 122 and ops['gemv_bf16'].id == 134
    assert ops['attn_decode_part'].arity == 18 and ops['adamw'].arity == 13 and ops['matmul_tile'].arity == 13
    assert len({o.id for o in ops.values()}) == len(ops)
    assert [a.optional for a in ops['embedding_fwd'].args][:4] == [False, False, True, False]
    assert all(o.arity <= abi.MAX_ARGS for o in ops.values())


def test_c_abi_exports_every_declared_symbol(kvm_lib):
    from kvm_b200.executor import SYMBOLS, lib
    header = (ROOT / 'include' / 'kvm_b200.h').read_text()
    declared = set(re.findall(r'\b(kvm_[a-z_0-9]+)\s*\(', header))
    assert declared == set(SYMBOLS), declared ^ set(SYMBOLS)
    L = lib()
    for name in declared:
        assert hasattr(L, name), name
    ops = abi.load_ops()
    for o in ops.values():          # the library's registry is the same text
        assert L.kvm_op_arity(o.id) == o.arity and L.kvm_op_name(o.id).decode() == o.name
    assert L.kvm_op_arity(64) == -1 and L.kvm_err_name(7) == b'VERSION_GAP' and L.kvm_err_name(1005) == b'E_TOKEN'


def test_executor_fails_loudly_without_gpu(kvm_lib):
    import torch
    if torch.cuda.is_available():
        pytest.skip('a GPU is present')
    from kvm_b200.executor import Executor, KvmError
    with pytest.raises(KvmError):
        Executor()


def _spec():
    return {'variables': ['weights'], 'buffers': [{'name': 'x', 'rows': 1, 'cols': 8, 'init': {'kind': 'values', 'values': list(range(8))}},
                                                  {'name': 'y', 'rows': 1, 'cols': 8}],
            'graphs': [{'name': 'g', 'tasks': [
                {'id': 'a', 'op': 'scale', 'args': {'x': 'x', 'out': 'y', 'alpha': 2.0, 'n': 8}, 'publishes': 'weights'},
                {'id': 'b', 'op': 'add', 'args': {'a': 'x', 'b': 'y', 'out': 'y', 'n': 8}, 'after': ['a'], 'priority': 3, 'reads': [{'var': 'weights', 'policy': 'at_least', 'version': 1}]},
                {'id': 'c', 'op': 'noop', 'after': ['b'], 'publishes': 'weights'}]}]}


def test_compile_spec_versions_and_roundtrip(tmp_path):
    b = compile_spec(_spec())
    assert validate(b) == ''
    t = b.tasks
    assert t['pub_ver'].tolist() == [1, 0, 2] and t['wait_var'].tolist() == [-1, 0, -1] and t['wait_ver'][1] == 1
    assert t['indegree'].tolist() == [0, 1, 1] and b.metadata['initial_ready'] == [0] and b.metadata['final_versions'] == {'weights': 2}
    b.write(tmp_path / 'bundle')
    b2 = load_bundle(tmp_path / 'bundle')
    assert np.array_equal(b2.tasks, b.tasks) and np.array_equal(b2.succ, b.succ) and np.array_equal(b2.args, b.args)
    vm = VM(b2).run()
    assert vm.buffer('y').a.reshape(-1).tolist() == [3.0 * i for i in range(8)] and vm.versions == {0: 2}
    assert (vm.exec_count == 1).all() and np.array_equal(vm.observed, b.tasks['indegree'])


@pytest.mark.parametrize('mutate, msg', [
    (lambda s: s['graphs'][0]['tasks'][0].update(op='nope'), 'unknown op'),
    (lambda s: s['graphs'][0]['tasks'][0]['args'].update(x='zz'), 'undeclared buffer'),
    (lambda s: s['graphs'][0]['tasks'][1].update(after=['zz']), 'unknown task'),
    (lambda s: s['graphs'][0]['tasks'][0].update(priority=40), 'priority'),
    (lambda s: s['graphs'][0]['tasks'][1]['reads'][0].update(version=9), 'never be satisfied'),
    (lambda s: s['graphs'][0]['tasks'][0]['args'].pop('out'), 'missing'),
    (lambda s: s['buffers'].append({'name': 'x', 'rows': 1, 'cols': 1}), 'duplicate buffer'),
])
def test_compile_errors(mutate, msg):
    s = _spec()
    mutate(s)
    with pytest.raises(CompileError, match=msg):
        compile_spec(s)


def test_validate_catches_malformed_bundles():
    b = compile_spec(_spec())
    def broken(f):
        c = Bundle(b.tasks.copy(), b.succ.copy(), b.args.copy(), b.metadata)
        f(c)
        return validate(c)
    assert 'bad op_id' in broken(lambda c: c.tasks['op_id'].__setitem__(0, 77))
    assert 'takes' in broken(lambda c: c.tasks['args_words'].__setitem__(0, 3))
    assert 'indegree' in broken(lambda c: c.tasks['indegree'].__setitem__(2, 0))
    assert 'buffer index' in broken(lambda c: c.args.__setitem__(0, 9))
    assert 'cycle' in broken(lambda c: (c.succ.__setitem__(1, 0), c.tasks['indegree'].__setitem__(0, 1), c.tasks['indegree'].__setitem__(2, 0)))
    assert 'version variable' in broken(lambda c: c.tasks['pub_var'].__setitem__(0, 5))


def test_graph_dataflow_orders_raw_war_waw():
    g = Graph('t')
    g.buffer('a', 4, 4), g.buffer('b', 4, 4)
    w0 = g.task('fill', {'x': 'a', 'value': 1.0, 'n': 16}, [], ['a'])
    r0 = g.task('copy', {'src': 'a', 'dst': 'b', 'n': 16}, [('a', (0, 2))], ['b'])
    w1 = g.task('fill', {'x': 'a', 'value': 2.0, 'n': 8}, [], [('a', (0, 2))])          # WAR on r0, WAW on w0
    r1 = g.task('copy', {'src': 'a', 'dst': 'b', 'n': 16}, [('a', (2, 4))], ['b'])       # RAW on w0 only (rows 2..4), WAW on r0
    assert g.preds[r0] == [w0] and g.preds[w1] == [w0, r0] and g.preds[r1] == [w0, r0]
    assert validate(g.to_bundle()) == ''


def test_training_graph_is_order_independent():
    """Dataflow completeness: any topological order of the emitted graph gives bit-identical state (the reference checks its
    frontend the same way, frontend/mvmfe/refvm.py:1-6)."""
    b = build_training(preset('gpt_micro'), 2).to_bundle()
    base = VM(b).run()
    rng = np.random.default_rng(3)
    t = b.tasks
    for trial in range(2):
        vm = VM(b)
        rem = t['indegree'].astype(np.int64).copy()
        ready = list(np.flatnonzero(rem == 0))
        while ready:
            i = int(ready.pop(int(rng.integers(len(ready)))))
            vm.run_task(i)
            for s in b.succ[t['succ_off'][i]:t['succ_off'][i] + t['succ_cnt'][i]]:
                rem[s] -= 1
                if rem[s] == 0:
                    ready.append(int(s))
        for x, y in zip(vm.bufs, base.bufs):
            assert np.array_equal(x.a.view(np.uint32), y.a.view(np.uint32))


def test_token_stream_data_parallel_split():
    cfg = preset('gpt_micro')
    ids_all, tgt_all = token_stream(cfg, 4, 0, 1)
    N = cfg.tokens
    for r in range(2):
        ids, tgt = token_stream(cfg, 2, r, 2)
        for s in range(2):        # rank r takes microbatch r of each group of 2
            assert np.array_equal(ids[s * N:(s + 1) * N], ids_all[(2 * s + r) * N:(2 * s + r + 1) * N])
    assert ((ids_all >= 0) & (ids_all < cfg.vocab)).all()
    assert np.array_equal(ids_all.reshape(-1, cfg.seq)[:, 1:], tgt_all.reshape(-1, cfg.seq)[:, :-1])


def test_flat_chunks_never_overlap():
    g = Graph('t')
    g.buffer('w', 768, 50304), g.buffer('v', 50304, 768), g.buffer('s', 1, 100000)
    for buf in ('w', 'v', 's'):
        ch = g.flat_chunks(buf, 262144)
        assert ch[0][0] == 0 and ch[-1][1] == g.buffers[buf]['rows'] * g.buffers[buf]['cols'] and all(a[1] == b[0] for a, b in zip(ch, ch[1:]))
        regs = [g.region_of(buf, *c) for c in ch]
        for (r0, c0), (r1, c1) in zip(regs, regs[1:]):
            assert r0[1] <= r1[0] or (r0 == r1 and c0[1] <= c1[0])


def test_mlp_graph_components_and_oracle_loss_falls():
    """The multi-MLP graph: one connected component per model (the shared input batches are only read), and on the oracle the
    momentum-SGD steps lower each model's loss."""
    from kvm_b200.workloads.mlp import build_mlps, preset
    from oracle.vm_np import VM
    c = preset('mlp_small')
    b = build_mlps(c, 6).to_bundle()
    validate(b)
    nt = len(b.tasks)
    parent = list(range(nt))

    def find(x):
        while parent[x] != x:
            parent[x] = parent[parent[x]]
            x = parent[x]
        return x
    for t in range(nt):
        o, n = int(b.tasks['succ_off'][t]), int(b.tasks['succ_cnt'][t])
        for s in b.succ[o:o + n]:
            parent[find(t)] = find(int(s))
    assert len({find(t) for t in range(nt)}) == len(c.widths)
    vm = VM(b).run()
    for mi in range(len(c.widths)):
        losses = [float(vm.buffer(f'm{mi}.loss.{s}').a[0, 0]) for s in range(6)]
        assert losses[-1] < losses[0], losses


def test_decode_phases_fit_whole_waves():
    """Balanced decode graph: the GEMV tasks of every concurrent phase of a layer fit the SM count (no straggler wave)."""
    from kvm_b200.workloads.decode import build_decode, preset
    import collections
    c = preset('qwen3_8b', layers=1, vocab=4096)
    names = build_decode(c).to_bundle(check=False).metadata['task_names']
    cnt = collections.Counter(n.split('.')[2] for n in names if '.l0.' in n and 'join' not in n)
    assert cnt['q'] + cnt['k'] + cnt['v'] <= c.workers and cnt['gate'] + cnt['up'] <= c.workers and cnt['o'] <= c.workers and cnt['down'] <= c.workers
    assert cnt['part'] == c.kv_heads * c.splits and cnt['merge'] == c.kv_heads


# ---- the C library's own host check, without a GPU (what kvm_submit runs before anything reaches a device) ---------------------
def _c_validate(b, nbufs=None, nvars=64):
    from kvm_b200.executor import validate_batch
    return validate_batch(b.tasks, b.succ, b.args, len(b.buffers) if nbufs is None else nbufs, nvars)


def test_c_validate_negatives(kvm_lib):
    b = compile_spec(_spec())
    assert _c_validate(b) == ''
    def broken(f, **kw):
        c = Bundle(b.tasks.copy(), b.succ.copy(), b.args.copy(), b.metadata)
        f(c)
        return _c_validate(c, **kw)
    assert 'bad op_id' in broken(lambda c: c.tasks['op_id'].__setitem__(0, 77))
    assert 'takes' in broken(lambda c: c.tasks['args_words'].__setitem__(0, 3))
    assert 'args range' in broken(lambda c: c.tasks['args_off'].__setitem__(0, 10 ** 6))
    assert 'successor range' in broken(lambda c: c.tasks['succ_cnt'].__setitem__(0, 99))
    assert 'successor' in broken(lambda c: c.succ.__setitem__(0, 17))
    assert 'priority' in broken(lambda c: c.tasks['priority'].__setitem__(0, 32))
    assert 'indegree' in broken(lambda c: c.tasks['indegree'].__setitem__(2, 0))
    assert 'buffer index' in broken(lambda c: c.args.__setitem__(0, 9))
    assert 'buffer index' in broken(lambda c: None, nbufs=1)
    assert 'cycle' in broken(lambda c: (c.succ.__setitem__(1, 0), c.tasks['indegree'].__setitem__(0, 1), c.tasks['indegree'].__setitem__(2, 0)))
    assert 'version variable' in broken(lambda c: c.tasks['pub_var'].__setitem__(0, 5), nvars=4)
    assert 'wait_ver' in broken(lambda c: c.tasks['pub_ver'].__setitem__(0, 0))
    assert 'publishes itself' in broken(lambda c: (c.tasks['wait_var'].__setitem__(0, 0), c.tasks['wait_ver'].__setitem__(0, 1)))
    # a waiter whose only possible publisher depends on it: b waits for version 2, which c publishes, and c runs after b
    assert 'version-wait cycle' in broken(lambda c: c.tasks['wait_ver'].__setitem__(1, 2))


def test_corrupted_bundles_are_rejected_on_the_host(kvm_lib):
    """Seeded corruption of a valid training bundle (the reference's tests/litmus/fuzz.py does this to bundle files): random
    words of the descriptor table, successor list and argument words are overwritten.  The host check must answer every time
    (no crash, no hang) and must reject every mutant that changes the graph's structure; whatever it accepts is still a
    well-formed program (indices in range, acyclic, indegrees equal to in-edges), which the Python twin confirms."""
    b = build_training(preset('gpt_micro'), 1).to_bundle()
    assert _c_validate(b) == ''
    rng = np.random.default_rng(7)
    rejected = 0
    for trial in range(300):
        c = Bundle(b.tasks.copy(), b.succ.copy(), b.args.copy(), b.metadata)
        which = trial % 3
        if which == 0:
            words = c.tasks.view(np.int32).reshape(-1)
            field = int(rng.integers(0, 12))            # op_id .. pub_ver
            i = int(rng.integers(0, len(c.tasks))) * 16 + field
            words[i] = int(rng.choice([-1, -2, 0, 1, 77, 1 << 20, -(1 << 31), (1 << 31) - 1, int(rng.integers(-1000, 1000))]))
            changed = True
        elif which == 1:
            i = int(rng.integers(0, len(c.succ)))
            old = int(c.succ[i])
            c.succ[i] = int(rng.choice([-1, len(c.tasks), 1 << 20, int(rng.integers(0, len(c.tasks)))]))
            changed = int(c.succ[i]) != old
        else:
            i = int(rng.integers(0, len(c.args)))
            old = int(c.args[i])
            c.args[i] = int(rng.choice([-2, len(c.buffers), 1 << 20, -(1 << 31)]))
            changed = False                               # a scalar argument may take any value: the device op range-checks it
        msg = _c_validate(c, nvars=len(b.metadata['variables']))
        py = validate(c)
        assert (msg == '') == (py == ''), (trial, msg, py)
        if msg:
            rejected += 1
        elif changed and which == 1:
            raise AssertionError(f'trial {trial}: a rewired successor was accepted')
    assert rejected > 150


def test_command_line_runner_usage_and_registry_without_a_gpu(kvm_lib):
    """The kvm_exec tool (reference CLI contract: exit 2 on usage errors) and the registry it was built with, arities included."""
    import subprocess
    from kvm_b200 import abi, build
    cli = build.build_cli()
    assert subprocess.run([str(cli)], capture_output=True).returncode == 2
    assert subprocess.run([str(cli), '--no-such-flag', 'x'], capture_output=True).returncode == 2
    r = subprocess.run([str(cli), '--check-ops'], capture_output=True, text=True)
    rows = [line.split() for line in r.stdout.splitlines()]
    assert r.returncode == 0
    assert {int(w[0]): (w[1], int(w[3])) for w in rows} == {o.id: (o.name, len(o.args)) for o in abi.load_ops().values()}
    # a bundle directory cannot run here: the tool says why on stderr and exits 1 without a result line
    r = subprocess.run([str(cli), '/nonexistent/bundle'], capture_output=True, text=True)
    assert r.returncode == 1 and r.stdout == '' and r.stderr
