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
        self._joins = {}
        self._wver = {}
        self.join_threshold = 24

    # ---- declarations
    def buffer(self, name, rows, cols, dtype='f32', init=None):
        if name in self.buffers:
            b = self.buffers[name]
            assert (b['rows'], b['cols'], b['dtype']) == (rows, cols, dtype), f'buffer {name} redeclared with another shape'
            return name
        self.buffers[name] = {'name': name, 'rows': int(rows), 'cols': int(cols), 'dtype': dtype,
                              'init': init or {'kind': 'fill', 'value': 0}}
        self._w[name], self._r[name] = _Records(), _Records()
        self._wver[name] = 0
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

    def data(self, name, values: np.ndarray, dtype='f32'):
        """A buffer initialised from an array (2-D), carried as a `file` init: raw little-endian f32 / i32 / bf16 bits."""
        values = np.atleast_2d(values)
        rel = f'data/{name}.bin'
        if dtype == 'bf16':
            u = np.ascontiguousarray(values, dtype=np.float32).view(np.uint32)
            raw = ((u + np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1))) >> np.uint32(16)).astype('<u2').tobytes()
        else:
            raw = np.ascontiguousarray(values, dtype='<i4' if dtype == 'i32' else '<f4').tobytes()
        self.blobs[rel] = raw
        return self.buffer(name, values.shape[0], values.shape[1], dtype, {'kind': 'file', 'path': rel})

    def variable(self, name):
        if name not in self.variables:
            self.variables.append(name)
            self._pubs[name] = 0
        return name

    def rows_of(self, buf, e0, e1):
        """Row range covering the flat element range [e0,e1) of `buf`."""
        c = self.buffers[buf]['cols']
        return (e0 // c, -(-e1 // c))

    def region_of(self, buf, e0, e1):
        """(rows, cols) region of the flat range [e0,e1): exact when it is whole rows or lies inside one row."""
        c = self.buffers[buf]['cols']
        if e0 // c == (e1 - 1) // c:
            return (e0 // c, e0 // c + 1), (e0 % c, (e1 - 1) % c + 1)
        return (e0 // c, -(-e1 // c)), ALL

    def flat_chunks(self, buf, target):
        """Flat ranges [e0,e1) of about `target` elements covering `buf`, cut on row boundaries (or inside single rows when a row
        is longer than the target), so neighbouring chunks never share a region and get no false dependency."""
        rows, c = self.buffers[buf]['rows'], self.buffers[buf]['cols']
        out = []
        if c >= 2 * target:
            per = -(-c // -(-c // target))
            per = -(-per // 8) * 8
            for r in range(rows):
                for c0 in range(0, c, per):
                    out.append((r * c + c0, r * c + min(c0 + per, c)))
        else:
            per = max(1, target // c)
            for r0 in range(0, rows, per):
                out.append((r0 * c, min(r0 + per, rows) * c))
        return out

    # ---- emission
    def task(self, op, args, reads=(), writes=(), priority=0, name=None, publishes=None, after=(), quiet_reads=()):
        """reads / writes: iterables of (buffer, (r0, r1), (c0, c1)); a buffer name alone means the whole buffer.
        quiet_reads are recorded for later writers (write-after-read) but add no edge now: the caller orders them through `after`
        (a join task that already waits for their producers)."""
        spec = self.ops[op]
        tid = len(self.tasks)
        deps = set(after)
        norm = lambda acc: [(a, ALL, ALL) if isinstance(a, str) else (a[0], a[1], a[2] if len(a) > 2 else ALL) for a in acc if a is not None and a[0] is not None]
        reads, writes, quiet_reads = norm(reads), norm(writes), norm(quiet_reads)
        for buf, (r0, r1), (c0, c1) in reads:
            w = self._w[buf]
            if w.n:
                prod = w.a[:w.n][w.overlapping(r0, r1, c0, c1), 4]
                if len(prod) > self.join_threshold:
                    # many producers of one region, usually shared by many readers: a noop join waits for them once
                    key = (buf, r0, r1, c0, c1, self._wver[buf])
                    if key not in self._joins:
                        self._joins[key] = len(self.tasks)
                        self.tasks.append({'name': f'join{len(self._joins)}:{buf}', 'op': self.ops['noop'], 'args': {}, 'priority': int(priority),
                                           'deadline_us': -1, 'pub': None, 'wait': None, 'gi': 0, 'publishes': None})
                        self.preds.append(sorted(set(prod.tolist())))
                        tid = len(self.tasks)
                    deps.add(self._joins[key])
                else:
                    deps.update(prod.tolist())
        for buf, (r0, r1), (c0, c1) in writes:
            w, r = self._w[buf], self._r[buf]
            ws = w.a[:w.n][w.overlapping(r0, r1, c0, c1)] if w.n else w.a[:0]
            deps.update(ws[:, 4].tolist())
            if r.n:
                rs = r.a[:r.n][r.overlapping(r0, r1, c0, c1)]
                if len(rs) and len(ws):
                    # a reader R is already ordered before this write if some overlapping earlier writer W was emitted after R
                    # and touched R's region (W then carries the edge R -> W, and W -> this task was just added)
                    covered = ((ws[None, :, 4] > rs[:, None, 4]) & (ws[None, :, 0] < rs[:, None, 1]) & (ws[None, :, 1] > rs[:, None, 0]) &
                               (ws[None, :, 2] < rs[:, None, 3]) & (ws[None, :, 3] > rs[:, None, 2])).any(axis=1)
                    rs = rs[~covered]
                deps.update(rs[:, 4].tolist())
        deps.discard(tid)
        for buf, (r0, r1), (c0, c1) in writes:
            self._w[buf].drop_covered(r0, r1, c0, c1)
            self._r[buf].drop_covered(r0, r1, c0, c1)
            self._w[buf].add(r0, r1, c0, c1, tid)
            self._wver[buf] += 1
        for buf, (r0, r1), (c0, c1) in reads + quiet_reads:
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

    def to_bundles_split(self, split_at: int):
        """Two bundles over the same buffer table: tasks [0, split_at) and [split_at, end). The second is meant to run after the
        first has finished entirely (a collective sits between them), so its edges from first-half tasks are dropped."""
        import copy
        first, second = copy.copy(self), copy.copy(self)
        first.tasks, first.preds = self.tasks[:split_at], self.preds[:split_at]
        first._pubs = {v: sum(1 for t in first.tasks if t['publishes'] == v) for v in self.variables}
        second.tasks = [dict(t) for t in self.tasks[split_at:]]
        second.preds = [[p - split_at for p in ps if p >= split_at] for ps in self.preds[split_at:]]
        base = dict(first._pubs)
        for t in second.tasks:      # publishes of the second half are numbered from 1 again: it is its own batch on its own handle
            if t['pub']:
                t['pub'] = (t['pub'][0], t['pub'][1] - base[t['pub'][0]])
        second._pubs = {v: self._pubs[v] - base[v] for v in self.variables}
        return first.to_bundle(), second.to_bundle()

    def to_bundles_multi(self, cuts):
        """One bundle per segment [cuts[i], cuts[i+1]) over the same buffer table, to be run one after the other (an exchange with
        other ranks sits between them): edges from earlier segments are dropped.  For graphs without version publishes."""
        import copy
        assert not any(t['pub'] for t in self.tasks), 'segments of a graph with publishes need renumbering'
        out, ends = [], list(cuts[1:]) + [len(self.tasks)]
        for a, b in zip(cuts, ends):
            seg = copy.copy(self)
            seg.tasks = [dict(t) for t in self.tasks[a:b]]
            seg.preds = [[p - a for p in ps if p >= a] for ps in self.preds[a:b]]
            out.append(seg.to_bundle())
        return out

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
