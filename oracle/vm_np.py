"""CPU oracle: a bundle interpreter over oracle.ops_np.  TEST INFRASTRUCTURE, not product code.

Restates the reference's CPU VM for one bundle (`runtime/workload_vm.py:60-286`): buffers are materialised from their
init specs (fill / values / seeded / file), tasks run once each when all in-bundle predecessors have finished and
`version[wait_var] >= wait_ver`; a finishing task with `pub_var` sets `version[pub_var] = pub_ver`, which must be the
old version + 1 (`include/mvm_task_abi.h:20-23`).  The run records, per task, how often it executed and how many
predecessor completions it observed, which is what "completion sets and dependency counts match" is checked against.
"""
from __future__ import annotations

import heapq

import numpy as np

from kvm_b200 import abi
from kvm_b200.bundle import Bundle
from kvm_b200.initgen import seeded_values

from . import ops_np
from .ops_np import BF16, I32, Buf, bf16_round


class VMError(RuntimeError):
    pass


def materialize(bundle: Bundle, b: dict) -> Buf:
    rows, cols, dt, init = b['rows'], b['cols'], b['dtype'], b['init']
    np_dt = np.int32 if dt == I32 else np.float32
    kind = init['kind']
    if kind == 'fill':
        a = np.full((rows, cols), init['value'], dtype=np_dt)
    elif kind == 'values':
        a = np.array(init['values'], dtype=np_dt).reshape(rows, cols)
    elif kind == 'seeded':
        a = seeded_values(init['seed'], rows * cols, init['draws'], init['bias'], init['coef']).reshape(rows, cols)
    elif kind == 'file':
        raw = bundle.init_bytes(b)
        if dt == BF16:
            a = (np.frombuffer(raw, '<u2').astype(np.uint32) << 16).view(np.float32).reshape(rows, cols).copy()
        else:
            a = np.frombuffer(raw, '<i4' if dt == I32 else '<f4').reshape(rows, cols).copy()
    else:
        raise VMError(f"buffer {b['name']!r}: unknown init kind {kind!r}")
    if dt == BF16:
        a = bf16_round(a)
    return Buf(np.ascontiguousarray(a), dt)


class VM:
    def __init__(self, bundle: Bundle, exact_matmul: bool = True, buffers: list | None = None, lazy: bool = False, zeros: bool = False, f64: bool = False):
        self.bundle = bundle
        self.exact = exact_matmul
        self.f64 = f64          # all-double rerun (oracle/f64.py): same ops without the float32 / bf16 rounding, float64 buffers
        self.opsmod = ops_np
        if f64:
            from .f64 import ops_f64
            self.opsmod = ops_f64()
        self.zeros = zeros      # timing-only mode: True = every buffer starts as zeros instead of its init; a callable(spec) -> array supplies other stand-in values
        # lazy=True materialises a buffer at its first use (bounded timing samples touch a fraction of a large model)
        self.bufs = buffers if buffers is not None else [None if lazy else materialize(bundle, b) for b in bundle.buffers]
        if f64:
            self.bufs = [b if b is None or b.dtype == I32 else Buf(b.a.astype(np.float64), b.dtype) for b in self.bufs]
        self.versions = {v['id']: v['base_version'] for v in bundle.metadata.get('variables', [])}
        self.ops = abi.ops_by_id()
        nt = len(bundle.tasks)
        self.exec_count = np.zeros(nt, np.int32)
        self.observed = np.zeros(nt, np.int32)
        self.order = []

    def buffer(self, name: str) -> Buf:
        for i, b in enumerate(self.bundle.buffers):
            if b['name'] == name:
                if self.bufs[i] is None:
                    self.bufs[i] = materialize(self.bundle, b)
                return self.bufs[i]
        raise KeyError(name)

    def run_task(self, i: int):
        t = self.bundle.tasks[i]
        op = self.ops[int(t['op_id'])]
        words = self.bundle.args[int(t['args_off']):int(t['args_off']) + int(t['args_words'])]
        bufs, scal = {}, {}
        for a, w in zip(op.args, words):
            if a.type == 'buf':
                if w != abi.ABSENT_BUF and self.bufs[int(w)] is None:
                    spec = self.bundle.buffers[int(w)]
                    if callable(self.zeros):
                        self.bufs[int(w)] = Buf(self.zeros(spec), spec['dtype'])
                    elif self.zeros:
                        self.bufs[int(w)] = Buf(np.zeros((spec['rows'], spec['cols']), np.int32 if spec['dtype'] == I32 else np.float32), spec['dtype'])
                    else:
                        self.bufs[int(w)] = materialize(self.bundle, spec)
                bufs[a.name] = None if w == abi.ABSENT_BUF else self.bufs[int(w)]
            elif a.type == 'i32':
                scal[a.name] = int(w)
            else:
                scal[a.name] = float(np.array([w], '<i4').view('<f4')[0])
        self.opsmod.OPS[op.name](bufs, scal, exact_matmul=self.exact)

    def run(self, subset=None, time_limit=None):
        """Run every task (or stop after `subset` tasks / `time_limit` seconds, for bounded timing samples). Returns self."""
        import time
        t_end = None if time_limit is None else time.perf_counter() + time_limit
        t = self.bundle.tasks
        nt = len(t)
        rem = t['indegree'].astype(np.int64).copy()
        so, sc = t['succ_off'], t['succ_cnt']
        ready = [(-int(t['priority'][i]), int(i)) for i in np.flatnonzero(rem == 0)]
        heapq.heapify(ready)
        parked, done = [], 0
        while ready or parked:
            if not ready:
                raise VMError(f'deadlock: {len(parked)} tasks parked on versions nobody publishes')
            _, i = heapq.heappop(ready)
            wv = int(t['wait_var'][i])
            if wv >= 0 and self.versions[wv] < int(t['wait_ver'][i]):
                parked.append(i)
                continue
            self.run_task(i)
            self.exec_count[i] += 1
            self.order.append(i)
            done += 1
            pv = int(t['pub_var'][i])
            if pv >= 0:
                if int(t['pub_ver'][i]) != self.versions[pv] + 1:
                    raise VMError(f'task {i}: VERSION_GAP publishing {int(t["pub_ver"][i])} over {self.versions[pv]}')
                self.versions[pv] = int(t['pub_ver'][i])
                still = []
                for j in parked:
                    if self.versions[int(t['wait_var'][j])] >= int(t['wait_ver'][j]):
                        heapq.heappush(ready, (-int(t['priority'][j]), j))
                    else:
                        still.append(j)
                parked = still
            for s in self.bundle.succ[int(so[i]):int(so[i]) + int(sc[i])]:
                s = int(s)
                rem[s] -= 1
                self.observed[s] += 1
                if rem[s] == 0:
                    heapq.heappush(ready, (-int(t['priority'][s]), s))
            if (subset is not None and done >= subset) or (t_end is not None and time.perf_counter() >= t_end):
                break
        if subset is None and time_limit is None and done != nt:
            raise VMError(f'{done}/{nt} tasks ran')
        return self
