"""Host-side structure of the one-launch multi-GPU forms (no GPU, no threads): who owns which gradient chunk, where every store
lands, which flag word announces it.  The data path itself is covered by the threaded oracle ranks in test_dp_gloo.py /
test_tp_gloo.py and on the device by tests/test_gpu_parallel_one_gpu.py."""
import numpy as np
import pytest

from kvm_b200 import abi
from kvm_b200.bundle import validate
from kvm_b200.workloads.decode import build_decode_tp, preset as decode_preset
from kvm_b200.workloads.gpt import build_training, dp_exchange_layout, param_shapes, preset

OPS = abi.load_ops()


def _tasks(bundle, op):
    """[(task index, {argument name: value})] of the tasks of one op."""
    spec = OPS[op]
    out = []
    for i in np.nonzero(bundle.tasks['op_id'] == spec.id)[0]:
        off = int(bundle.tasks['args_off'][i])
        words = bundle.args[off:off + len(spec.args)]
        out.append((int(i), {a.name: int(w) for a, w in zip(spec.args, words)}))
    return out


def _name(bundle, idx):
    return bundle.buffers[idx]['name']


@pytest.mark.parametrize('world', [2, 4, 8])
def test_gradient_exchange_covers_every_chunk_exactly_once(world):
    cfg = preset('gpt_micro')
    arena, n_arena, chunks, width, owned = dp_exchange_layout(cfg, world)
    # the arena: every parameter once, 64-element aligned, no overlap
    spans = sorted((off, off + r * c) for (name, r, c, _, _), off in zip(param_shapes(cfg), arena.values()))
    assert all(a % 64 == 0 for a, _ in spans) and all(spans[i][1] <= spans[i + 1][0] for i in range(len(spans) - 1)) and spans[-1][1] <= n_arena
    assert owned == -(-len(chunks) // world) and width >= max(e1 - e0 for _, e0, e1 in chunks) and width % 4 == 0
    landed = {p: [] for p in range(world)}          # rank -> [(arena offset, n)] of the sums stored into its arena by the owners
    for rank in range(world):
        b = build_training(cfg, 1, rank=rank, world=world, stream_steps=2, dp_fused=True).to_bundle()
        assert validate(b) == ''                      # the host check (first problem as text, empty when there is none)
        assert [s['name'] for s in b.buffers[:4]] == ['dp.arena', 'dp.inbox', 'dp.flag', 'dp.gflag']
        mine = [k for k in range(len(chunks)) if k % world == rank]
        sums, puts, waits = _tasks(b, 'peer_wait_sum'), _tasks(b, 'peer_put_signal'), _tasks(b, 'peer_wait')
        assert len(sums) == len(mine) and len(waits) == len(chunks) - len(mine)
        assert len(puts) == len(mine) * (world - 1) + len(chunks) - len(mine)
        for (_, a), k in zip(sums, mine):
            name, e0, e1 = chunks[k]
            assert _name(b, a['partial']) == _name(b, a['out']) == 'g.' + name and a['p_off'] == a['o_off'] == e0 and a['n'] == e1 - e0
            assert a['row0'] == (k // world) * world and a['rank'] == rank and a['world'] == world and _name(b, a['seq']) == 'opt_step'
        seen = set()
        for _, a in puts:
            dst = _name(b, a['dst'])
            p = int(dst.split('.')[1][4:])
            assert p != rank and _name(b, a['flag']).startswith(f'dp.peer{p}.')
            if dst.endswith('.inbox'):                # a partial chunk for its owner
                row, col = divmod(a['dst_off'], width)
                assert col == 0 and row % world == rank and a['var'] == row and _name(b, a['flag']).endswith('.flag')
                k = (row // world) * world + p
                assert chunks[k][2] - chunks[k][1] == a['n'] and a['src_off'] == chunks[k][1] and (p, row) not in seen
                seen.add((p, row))
            else:                                     # a summed chunk for a peer's arena
                assert dst.endswith('.arena') and _name(b, a['flag']).endswith('.gflag')
                name, e0, e1 = chunks[a['var']]
                assert a['var'] % world == rank and a['dst_off'] == arena[name] + e0 and a['n'] == e1 - e0 and a['src_off'] == e0
                landed[p].append((a['dst_off'], a['n']))
        # the waits for the sums coming back run after the rank has sent its last chunk
        sent = [i for i, n in enumerate(b.metadata['task_names']) if n.endswith('dp.sent')]
        assert len(sent) == (1 if len(chunks) > len(mine) else 0)
        for i, a in waits:
            assert a['row0'] % world != rank and a['count'] == 1 and _name(b, a['flag']) == 'dp.gflag'
    for p in range(world):          # every chunk a rank does not own lands in its arena exactly once
        want = sorted((arena[n] + e0, e1 - e0) for k, (n, e0, e1) in enumerate(chunks) if k % world != p)
        assert sorted(landed[p]) == want


@pytest.mark.parametrize('world', [2, 4])
def test_tensor_parallel_exchange_sites(world):
    cfg = decode_preset('decode_tiny', kv_heads=max(2, world))
    sites = 2 * cfg.layers
    for rank in range(world):
        b = build_decode_tp(cfg, rank, world, exact=False, fused=True)[0].to_bundle()
        names = [s['name'] for s in b.buffers[:2 + 2 * (world - 1)]]
        assert names[:2] == ['tp.inbox', 'tp.flag'] and all(n.startswith('tp.peer') for n in names[2:])
        sums, puts = _tasks(b, 'peer_wait_sum'), _tasks(b, 'peer_put_signal')
        assert len(sums) == sites and len(puts) == sites * (world - 1)
        assert sorted(a['row0'] for _, a in sums) == [s * world for s in range(sites)]
        for _, a in puts:
            assert a['var'] % world == rank and a['dst_off'] == a['var'] * cfg.hidden and a['n'] == cfg.hidden


def test_c_validator_accepts_the_exchange_ops_and_rejects_a_short_argument_list():
    """The C library's host check (no GPU) knows the extension ops' arities from the same registry file."""
    from kvm_b200.executor import validate_batch
    b = build_training(preset('gpt_micro'), 1, rank=1, world=2, stream_steps=2, dp_fused=True).to_bundle()
    assert validate_batch(b.tasks, b.succ, b.args, len(b.buffers)) == ''
    t = b.tasks.copy()
    i = int(np.nonzero(t['op_id'] == OPS['peer_wait_sum'].id)[0][0])
    t['args_words'][i] -= 2            # the offsets are missing: an older caller's 12-word form
    assert 'arg' in validate_batch(t, b.succ, b.args, len(b.buffers)).lower()
    d = build_decode_tp(decode_preset('decode_tiny'), 0, 2, fused=True)[0].to_bundle()
    assert validate_batch(d.tasks, d.succ, d.args, len(d.buffers)) == ''
