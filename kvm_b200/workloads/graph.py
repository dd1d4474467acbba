"""Task-graph builder: ops are emitted as tile tasks that declare which buffer regions they read and write, and the
dependency edges follow from those regions (read-after-write, write-after-read, write-after-write), the same contract the
reference frontend's dataflow pass gives its emitter (`frontend/mvmfe/dataflow.py`, `FRONTEND.md:7-24`).  The result
is either the workload JSON the reference compiler accepts or, directly, an ABI v2 bundle.
"""
from __future__ import annotations

import numpy as np

from .. import abi
from ..bundle import Bundle, pack_bundle, validate

ALL = (0, 1 << 30)


class _Records:
    """Growable table of (r0, r1, c0, c1, task) access records of one buffer."""
    __slots__ = ('a', 'n')

    def __init__(self):
        self.a = np.empty((16, 5), np.int64)
        self.n = 0

    def overlapping(self, r0, r1, c0, c1):
        a = self.a[:self.n]
        return (a[:, 0] < r1) & (a[:, 1] > r0) & (a[:, 2] < c1) & (a[:, 3] > c0)

    def add(self, r0, r1, c0, c1, task):
        if self.n == len(self.a):
            self.a = np.concatenate([self.a, np.empty_like(self.a)])
        self.a[self.n] = (r0, r1, c0, c1, task)
        self.n += 1

    def drop_covered(self, r0, r1, c0, c1):
        a = self.a[:self.n]
        keep = ~((a[:, 0] >= r0) & (a[:, 1] <= r1) & (a[:, 2] >= c0) & (a[:, 3] <= c1))
        k = int(keep.sum())
        if k != self.n:
            self.a[:k] = a[keep]
            self.n = k


class Graph:
    def __init__(self, name='train'):
        self.name = name
        self.buffers: dict[str, dict] = {}
        self.variables: list[str] = []
        self.tasks: list[dict] = []
        self.preds: list[list[int]] = []
        self._w: dict[str, _Records] = {}
        self._r: dict[str, _Records] = {}
        self.blobs: dict[str, bytes] = {}
        self.ops = abi.load_ops()
        self._pubs = {}

    # ---- declarations
    def buffer(self, name, rows, cols, dtype='f32', init=None):
        if name in self.buffers:
            b = self.buffers[name]
            assert (b['rows'], b['cols'], b['dtype']) == (rows, cols, dtype), f'buffer {name} redeclared with another shape'
            return name
        self.buffers[name] = {'name': name, 'rows': int(rows), 'cols': int(cols), 'dtype': dtype,
                              'init': init or {'kind': 'fill', 'value': 0}}
        self._w[name], self._r[name] = _Records(), _Records()
        return name

    def stream(self, name, values: np.ndarray, cols=1):
        """An i32 host data stream; long ones travel as a `file` init next to the bundle (as the reference frontend does)."""
        values = np.ascontiguousarray(values, dtype='<i4')
        rows = values.size // cols
        if values.size <= 4096:
            init = {'kind': 'values', 'values': [int(v) for v in values.reshape(-1)]}
        else:
            rel = f'data/{name}.bin'
            self.blobs[rel] = values.tobytes()
            init = {'kind': 'file', 'path': rel}
        return self.buffer(name, rows, cols, 'i32', init)

    def variable(self, name):
        if name not in self.variables:
            self.variables.append(name)
            self._pubs[name] = 0
        return name

    def rows_of(self, buf, e0, e1):
        """Row range covering the flat element range [e0,e1) of `buf`."""
        c = self.buffers[buf]['cols']
        return (e0 // c, -(-e1 // c))

    # ---- emission
    def task(self, op, args, reads=(), writes=(), priority=0, name=None, publishes=None, after=()):
        """reads / writes: iterables of (buffer, (r0, r1), (c0, c1)); a buffer name alone means the whole buffer."""
        spec = self.ops[op]
        tid = len(self.tasks)
        deps = set(after)
        norm = lambda acc: [(a, ALL, ALL) if isinstance(a, str) else (a[0], a[1], a[2] if len(a) > 2 else ALL) for a in acc if a is not None and a[0] is not None]
        reads, writes = norm(reads), norm(writes)
        for buf, (r0, r1), (c0, c1) in reads:
            w = self._w[buf]
            if w.n:
                deps.update(w.a[:w.n][w.overlapping(r0, r1, c0, c1), 4].tolist())
        for buf, (r0, r1), (c0, c1) in writes:
            for rec in (self._w[buf], self._r[buf]):
                if rec.n:
                    deps.update(rec.a[:rec.n][rec.overlapping(r0, r1, c0, c1), 4].tolist())
        deps.discard(tid)
        for buf, (r0, r1), (c0, c1) in writes:
            self._w[buf].drop_covered(r0, r1, c0, c1)
            self._r[buf].drop_covered(r0, r1, c0, c1)
            self._w[buf].add(r0, r1, c0, c1, tid)
        for buf, (r0, r1), (c0, c1) in reads:
            self._r[buf].add(r0, r1, c0, c1, tid)
        pub = None
        if publishes is not None:
            self.variable(publishes)
            self._pubs[publishes] += 1
            pub = (publishes, self._pubs[publishes])
        self.tasks.append({'name': name or f'{tid}:{op}', 'op': spec, 'args': dict(args), 'priority': int(priority),
                           'deadline_us': -1, 'pub': pub, 'wait': None, 'gi': 0, 'publishes': publishes})
        self.preds.append(sorted(deps))
        return tid

    # ---- outputs
    def _words(self, t, index):
        out = []
        for a in t['op'].args:
            v = t['args'].get(a.name)
            if a.type == 'buf':
                out.append(abi.ABSENT_BUF if v is None else index[v])
            elif a.type == 'i32':
                out.append(int(v))
            else:
                out.append(abi.f32_word(float(v)))
        return out

    def to_bundle(self, check=True) -> Bundle:
        from ..bundle import _parse_init
        index = {n: i for i, n in enumerate(self.buffers)}
        bufs = [{'name': b['name'], 'index': i, 'rows': b['rows'], 'cols': b['cols'], 'dtype': abi.DTYPES[b['dtype']],
                 'init': _parse_init(b['name'], b['init'], b['rows'], b['cols'], b['dtype'])} for i, b in enumerate(self.buffers.values())]
        variables = {n: {'name': n, 'id': i, 'base_version': 0} for i, n in enumerate(self.variables)}
        for t in self.tasks:
            t['words'] = self._words(t, index)
        pubs = [{'task': i, 'name': f"{self.name}/{t['name']}", 'var': variables[t['pub'][0]]['id'], 'version': t['pub'][1]}
                for i, t in enumerate(self.tasks) if t['pub']]
        named = [{**t, 'name': f"{self.name}/{t['name']}"} for t in self.tasks]
        tasks, succ, args, meta = pack_bundle(named, self.preds, bufs, variables, pubs, [], dict(self._pubs))
        b = Bundle(tasks, succ, args, meta, None, dict(self.blobs))
        if check:
            problem = validate(b)
            assert not problem, problem
        return b

    def to_spec(self) -> dict:
        """The same program as workload JSON (`FRAMEWORK.md:27-60` of the reference): what its compiler takes."""
        tasks = []
        for i, t in enumerate(self.tasks):
            d = {'id': t['name'], 'op': t['op'].name, 'args': {k: v for k, v in t['args'].items()}, 'priority': t['priority']}
            if self.preds[i]:
                d['after'] = [self.tasks[p]['name'] for p in self.preds[i]]
            if t['publishes']:
                d['publishes'] = t['publishes']
            tasks.append(d)
        bufs = []
        for b in self.buffers.values():
            d = {'name': b['name'], 'rows': b['rows'], 'cols': b['cols'], 'init': b['init']}
            if b['dtype'] != 'f32':
                d['dtype'] = b['dtype']
            bufs.append(d)
        return {'variables': list(self.variables), 'buffers': bufs, 'graphs': [{'name': self.name, 'tasks': tasks}]}
