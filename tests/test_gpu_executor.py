"""The executor itself on the GPU, through the C ABI: version waits and parking, publish errors, priority classes, seeded random
DAGs on 1 / 7 / 148 workers (exactly once, every predecessor observed, no task starts before a predecessor ended), device-seeded
buffers bit for bit, data-dependent op errors, and the resident-program semantics of kvm_submit / kvm_run.

What these mirror in the reference: tests/gpu/test_exec.cu suites `dag` (:283-318, random DAGs x grid sizes, ordered
timestamps), `versions` (:694-705) and `errors`, and tests/gpu/initgen_vectors.txt.  Failures are produced on the host side only
(a bundle whose wait nothing satisfies, a publish of the wrong version, a bad token id): every device wait is bounded and the
launch ends with a status.
"""
import json
from pathlib import Path

import numpy as np
import pytest

from kvm_b200 import abi

pytestmark = pytest.mark.gpu

G = Path(__file__).resolve().parent / 'golden'
OPS = abi.load_ops()


def raw_bundle(tasks):
    """tasks: list of dicts {op, args (words), after (indices), priority, wait (var, ver), pub (var, ver)} -> (descriptors, CSR
    successors, argument words) as kvm_submit takes them."""
    n = len(tasks)
    succs = [[] for _ in range(n)]
    for i, t in enumerate(tasks):
        for p in t.get('after', ()):
            succs[p].append(i)
    arr = np.zeros(n, abi.TASK_DTYPE)
    succ, args = [], []
    for i, t in enumerate(tasks):
        spec = OPS[t['op']]
        words = list(t.get('args', ()))
        assert len(words) == spec.arity, (t['op'], len(words), spec.arity)
        wait, pub = t.get('wait', (-1, 0)), t.get('pub', (-1, 0))
        arr[i] = (spec.id, len(succ), len(succs[i]), len(t.get('after', ())), t.get('priority', 0), -1, len(args), len(words), wait[0], wait[1], pub[0], pub[1], 0, 0, 0, 0)
        succ += succs[i]
        args += words
    return arr, np.array(succ, np.int32), np.array(args, np.int32)


def scale_task(x, out, alpha, e0, e1, **kw):
    return {'op': 'scale_flat', 'args': [x, out, abi.f32_word(alpha), e0, e1], **kw}


# ---- version variables ---------------------------------------------------------------------------------------------------------
def test_waiters_park_until_the_publisher_in_the_same_launch_runs(kvm_lib):
    """300 root tasks wait for version 1 of a variable that the LAST task of a 40-task chain publishes: they are released at
    once (no predecessors), find the version too low, park, and are woken by the publish.  Each doubles one cell of a buffer the
    chain's last task filled, so a waiter that ran early would read zeros."""
    from kvm_b200.executor import Executor
    with Executor(trace=True) as ex:
        x = ex.add_buffer(1, 512, 0, None)
        y = ex.add_buffer(1, 512, 0, None)
        n = ex.add_buffer(1, 64, 1, None)
        tasks = [{'op': 'spin', 'args': [200]}]
        for i in range(1, 40):
            tasks.append({'op': 'counter_inc', 'args': [n, 0, 1, 1], 'after': [i - 1]})
        tasks.append({'op': 'fill', 'args': [x, abi.f32_word(3.0), 512], 'after': [39], 'pub': (2, 1)})
        first_waiter = len(tasks)
        for i in range(300):
            tasks.append(scale_task(x, y, 2.0, i, i + 1, wait=(2, 1), priority=31))
        t, s, a = raw_bundle(tasks)
        ex.submit(t, s, a)
        res = ex.run()
        assert res.done == len(tasks) and ex.get_version(2) == 1
        execs, observed = ex.task_counts(len(tasks))
        assert (execs == 1).all() and np.array_equal(observed, t['indegree'])
        out = ex.read_buffer(y)[0]
        assert (out[:300] == 6.0).all() and (out[300:] == 0.0).all()
        st, en, _ = ex.trace(len(tasks))
        assert st[first_waiter:].min() >= en[40], 'a waiter started before the publisher had finished'
        # the same program again: the next window of the template (waits and publishes shift with the variable)
        res = ex.run()
        assert res.done == len(tasks) and ex.get_version(2) == 2


def test_wait_satisfied_across_launches_and_by_the_host(kvm_lib):
    from kvm_b200.executor import Executor
    with Executor() as ex:
        x = ex.add_buffer(1, 64, 0, 1.0)
        ex.set_version(5, 7)                                   # the host publishes: base version 7
        t, s, a = raw_bundle([scale_task(x, x, 2.0, 0, 64, wait=(5, 7), pub=(5, 8))])
        ex.submit(t, s, a)
        assert ex.run().done == 1 and ex.get_version(5) == 8
        ex.clear_tasks()
        # a second batch, compiled against version 8, waits for what the first launch published
        t, s, a = raw_bundle([scale_task(x, x, 3.0, 0, 64, wait=(5, 8))])
        ex.submit(t, s, a)
        assert ex.run().done == 1
        assert (ex.read_buffer(x) == 6.0).all()


def test_publish_of_a_skipped_version_is_a_clean_error(kvm_lib):
    """pub_ver must be old + 1 (include/mvm_task_abi.h:20-23): publishing 2 over 0 ends the launch with VERSION_GAP (code 7)."""
    from kvm_b200.executor import Executor
    with Executor() as ex:
        x = ex.add_buffer(1, 64, 0, 1.0)
        t, s, a = raw_bundle([scale_task(x, x, 2.0, 0, 64, pub=(0, 2))])
        ex.submit(t, s, a)
        res = ex.run(check=False)
        assert res.status == 7 and res.err_task == 0 and abi.err_name(res.status) == 'VERSION_GAP'


def test_a_wait_nothing_satisfies_runs_out_and_the_launch_ends(kvm_lib):
    """A bounded wait on the device: the parked task's version never comes, the stall limit (300 ms here) expires, every worker
    leaves, and the host gets TIMEOUT with the count of finished tasks; the handle stays usable."""
    from kvm_b200.executor import Executor
    with Executor(timeout_ms=300) as ex:
        x = ex.add_buffer(1, 64, 0, 1.0)
        t, s, a = raw_bundle([scale_task(x, x, 2.0, 0, 32), scale_task(x, x, 2.0, 32, 64, wait=(1, 1))])
        ex.submit(t, s, a)
        res = ex.run(check=False)
        assert res.status == 15 and res.done == 1, (res.status, res.done)          # KVM_ERR_TIMEOUT
        out = ex.read_buffer(x)[0]
        assert (out[:32] == 2.0).all() and (out[32:] == 1.0).all()
        ex.clear_tasks()
        t, s, a = raw_bundle([scale_task(x, x, 2.0, 32, 64)])
        ex.submit(t, s, a)
        assert ex.run().done == 1 and (ex.read_buffer(x) == 2.0).all()


# ---- priority classes -----------------------------------------------------------------------------------------------------------
def test_higher_priority_class_is_served_first(kvm_lib):
    """One root releases 240 short tasks of the lowest class and 240 of the highest in one go (low ones listed first); four
    workers then serve the queue: the high class is drained before the low one is touched, apart from the tasks that were
    handed out while the release was still in progress (at most a few per worker)."""
    from kvm_b200.executor import Executor
    workers = 4
    with Executor(trace=True, workers=workers) as ex:
        tasks = [{'op': 'spin', 'args': [50]}]
        tasks += [{'op': 'spin', 'args': [20], 'after': [0], 'priority': 0} for _ in range(240)]
        tasks += [{'op': 'spin', 'args': [20], 'after': [0], 'priority': 31} for _ in range(240)]
        t, s, a = raw_bundle(tasks)
        ex.submit(t, s, a)
        assert ex.run().done == len(tasks)
        st, en, _ = ex.trace(len(tasks))
        low, high = st[1:241], st[241:]
        assert np.median(high) < np.median(low)
        assert int((low < high.max()).sum()) <= 4 * workers, f'{int((low < high.max()).sum())} low-class tasks started before the last high-class one'


# ---- random DAGs ------------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize('workers', [1, 7, 148])
@pytest.mark.parametrize('seed', [0, 1, 2])
def test_random_dag_exactly_once_and_ordered(kvm_lib, workers, seed):
    from kvm_b200.executor import Executor
    rng = np.random.default_rng(1000 + seed)
    n = 1500
    with Executor(trace=True, workers=workers) as ex:
        cells = ex.add_buffer(1, n, 1, None)
        x = ex.add_buffer(1, n, 0, 1.0)
        tasks = []
        for i in range(n):
            width = int(rng.choice([0, 1, 2, 3, 8, 40]))
            lo = max(0, i - int(rng.choice([4, 60, 600])))
            after = sorted(set(int(p) for p in rng.integers(lo, i, size=min(width, i - lo)))) if i > lo else []
            kind = int(rng.integers(0, 3))
            prio = int(rng.integers(0, 32))
            if kind == 0:
                tasks.append({'op': 'noop', 'args': [], 'after': after, 'priority': prio})
            elif kind == 1:
                tasks.append({'op': 'counter_inc', 'args': [cells, i, i + 1, 1], 'after': after, 'priority': prio})
            else:
                tasks.append(scale_task(x, x, 2.0, i, i + 1, after=after, priority=prio))
        t, s, a = raw_bundle(tasks)
        ex.submit(t, s, a)
        for run in range(2):          # armed twice: the second launch must be as clean as the first
            res = ex.run()
            assert res.done == n
            execs, observed = ex.task_counts(n)
            assert (execs == 1).all() and np.array_equal(observed, t['indegree'])
            st, en, _ = ex.trace(n)
            assert (en >= st).all() and (st > 0).all()
            for i, tk in enumerate(tasks):
                for p in tk['after']:
                    assert st[i] >= en[p], f'task {i} started at {st[i]} before its predecessor {p} ended at {en[p]}'
        kinds = np.array([OPS_ID[tk['op']] for tk in tasks])
        assert np.array_equal(ex.read_buffer(cells)[0], np.where(kinds == 1, 2, 0))
        assert np.array_equal(ex.read_buffer(x)[0], np.where(kinds == 2, 4.0, 1.0).astype(np.float32))


OPS_ID = {'noop': 0, 'counter_inc': 1, 'scale_flat': 2}


# ---- seeded initialisation on the device ------------------------------------------------------------------------------------------
def test_device_seeded_buffers_match_the_reference_bit_patterns(kvm_lib):
    """kvm_add_buffer(SEEDED) against the bit patterns the reference's GPU test holds (tests/gpu/initgen_vectors.txt), f32
    storage bit for bit, and bf16 storage = the same values rounded to nearest even once."""
    from kvm_b200.executor import Executor, bf16_bits
    v = json.loads((G / 'vectors.json').read_text())
    with Executor() as ex:
        for case in v['initgen']:
            bias = float(np.array([int(case['bias_bits'], 16)], np.uint32).view(np.float32)[0])
            coef = float(np.array([int(case['coef_bits'], 16)], np.uint32).view(np.float32)[0])
            want = np.array([int(x, 16) for x in case['bits']], np.uint32)
            n = case['n']
            i = ex.add_buffer(1, n, 0, ('seeded', case['seed'], case['draws'], bias, coef))
            assert np.array_equal(ex.read_buffer(i).reshape(-1).view(np.uint32), want), case['seed']
            j = ex.add_buffer(1, n, 2, ('seeded', case['seed'], case['draws'], bias, coef))
            raw = np.empty(n, np.uint16)
            ex._check(ex.L.kvm_read_buffer_raw(ex._h, j, raw.ctypes.data, raw.nbytes, 0))
            assert np.array_equal(raw, bf16_bits(want.view(np.float32))), case['seed']


# ---- data-dependent op errors -------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize('op', ['embedding_fwd', 'gather_rows'])
def test_bad_token_in_any_row_is_reported(kvm_lib, op):
    """A token id outside the table in a row that thread 0 never touches (d = 64: thread 0 owns every 8th row) must still end
    the launch with E_TOKEN (the reference reports it from whichever thread meets it)."""
    from kvm_b200.executor import Executor
    d, rows, V = 64, 32, 50
    ids = np.arange(rows, dtype=np.int32) % V
    ids[13] = V + 5
    with Executor() as ex:
        b_ids = ex.add_buffer(rows, 1, 1, ids)
        tab = ex.add_buffer(V, d, 0, np.ones((V, d), np.float32))
        out = ex.add_buffer(rows, d, 0, None)
        if op == 'embedding_fwd':
            task = {'op': op, 'args': [b_ids, tab, -1, out, 0, rows, rows, d]}
        else:
            task = {'op': op, 'args': [tab, b_ids, out, 0, rows, d]}
        t, s, a = raw_bundle([task])
        ex.submit(t, s, a)
        res = ex.run(check=False)
        assert res.status == 1005 and res.err_a == V + 5 and res.err_b == 13, (res.status, res.err_a, res.err_b)


# ---- resident-program semantics -------------------------------------------------------------------------------------------------------
def test_submitted_batches_form_one_resident_program(kvm_lib):
    """submit(A); run; submit(B); run executes A, then A and B (the documented difference from the reference, where a batch
    runs once); kvm_clear_tasks starts a new program."""
    from kvm_b200.executor import Executor
    with Executor() as ex:
        n = ex.add_buffer(1, 2, 1, None)
        A = raw_bundle([{'op': 'counter_inc', 'args': [n, 0, 1, 1]}])
        B = raw_bundle([{'op': 'counter_inc', 'args': [n, 1, 2, 1]}])
        ex.submit(*A)
        assert ex.run().done == 1
        ex.submit(*B)
        res = ex.run()
        assert res.done == 2 and res.admitted == 2
        assert ex.read_buffer(n)[0].tolist() == [2, 1]
        ex.clear_tasks()
        ex.submit(*B)
        assert ex.run().done == 1
        assert ex.read_buffer(n)[0].tolist() == [2, 2]
        # a buffer added after kvm_rearm is seen by the next start (the device tables are prepared again)
        ex.rearm()
        m = ex.add_buffer(1, 4, 1, None)
        assert ex.run().done == 1 and ex.read_buffer(n)[0].tolist() == [2, 3]
        ex.clear_tasks()
        ex.submit(*raw_bundle([{'op': 'counter_inc', 'args': [m, 0, 4, 5]}]))
        assert ex.run().done == 1 and ex.read_buffer(m)[0].tolist() == [5, 5, 5, 5]
