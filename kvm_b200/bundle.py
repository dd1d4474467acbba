"""Workload JSON -> ABI v2 bundle, and the on-disk bundle directory (tasks.bin, successors.bin, args.bin, metadata.json).

Both formats are the reference's: the JSON schema is the one `runtime/compile_workload.py:624-691` accepts
({variables, buffers, graphs[{name, tasks[{id, op, args, after, priority, deadline_us, publishes, reads}]}]}) and the
directory is what its `write_bundle` (`runtime/compile_workload.py:694-713`) produces, so a bundle written by either
compiler loads in either executor.  Version planning (publish numbering, exact-read write-after-read edges, noop gates
for second and later waits) follows `_plan_versions` / `_lay_out` (`runtime/compile_workload.py:452-522`).
"""
from __future__ import annotations

import json
import math
from dataclasses import dataclass, field
from pathlib import Path

import numpy as np

from . import abi
from .initgen import seeded_params

INT32_MAX = 2**31 - 1


class CompileError(ValueError):
    """The workload is invalid; the message names the graph / task / argument at fault."""


def _need(cond, msg):
    if not cond:
        raise CompileError(msg)


@dataclass
class Bundle:
    tasks: np.ndarray                 # structured, abi.TASK_DTYPE
    succ: np.ndarray                  # int32
    args: np.ndarray                  # int32
    metadata: dict
    data_dir: Path | None = None      # where `file` inits are resolved
    blobs: dict = field(default_factory=dict)   # relative path -> bytes for `file` inits not yet on disk

    @property
    def buffers(self):
        return self.metadata['buffers']

    def write(self, out_dir) -> Path:
        out = Path(out_dir)
        out.mkdir(parents=True, exist_ok=True)
        self.tasks.tofile(out / 'tasks.bin')
        self.succ.astype('<i4').tofile(out / 'successors.bin')
        self.args.astype('<i4').tofile(out / 'args.bin')
        (out / 'metadata.json').write_text(json.dumps(self.metadata, separators=(',', ':')))
        for rel, data in self.blobs.items():
            (out / rel).parent.mkdir(parents=True, exist_ok=True)
            (out / rel).write_bytes(data)
        for b in self.buffers:
            if b['init']['kind'] == 'file' and b['init']['path'] not in self.blobs and self.data_dir is not None:
                src, dst = Path(self.data_dir) / b['init']['path'], out / b['init']['path']
                if src.resolve() != dst.resolve():
                    dst.parent.mkdir(parents=True, exist_ok=True)
                    dst.write_bytes(src.read_bytes())
        return out

    def init_bytes(self, b: dict) -> bytes | None:
        """Raw little-endian content of a `file` init."""
        rel = b['init']['path']
        if rel in self.blobs:
            return self.blobs[rel]
        return (Path(self.data_dir) / rel).read_bytes()


def load_bundle(bundle_dir) -> Bundle:
    d = Path(bundle_dir)
    meta = json.loads((d / 'metadata.json').read_text())
    _need(meta.get('abi_version') == abi.ABI_VERSION, f"{d}: abi_version {meta.get('abi_version')} != {abi.ABI_VERSION}")
    tasks = np.fromfile(d / 'tasks.bin', dtype=abi.TASK_DTYPE)
    succ = np.fromfile(d / 'successors.bin', dtype='<i4')
    args = np.fromfile(d / 'args.bin', dtype='<i4')
    _need(len(tasks) == meta['task_count'] and len(succ) == meta['edge_count'] and len(args) == meta['args_words'],
          f'{d}: file sizes disagree with metadata.json')
    return Bundle(tasks, succ, args, meta, d)


def validate(b: Bundle, nbufs: int | None = None, nvars: int | None = None) -> str:
    """'' if well formed, else the first problem: the host check the reference does in `MvmBundle::validate`
    (`mvm_exec.cu:141-208`): op ids, arities, ranges, buffer indices, indegree == in-edges, acyclic."""
    ops = abi.ops_by_id()
    t, nt = b.tasks, len(b.tasks)
    if nt == 0:
        return 'empty bundle'
    nbufs = len(b.buffers) if nbufs is None else nbufs
    nvars = len(b.metadata.get('variables', [])) if nvars is None else nvars
    for i in range(nt):
        op = ops.get(int(t['op_id'][i]))
        if op is None:
            return f"task {i}: bad op_id {int(t['op_id'][i])}"
        if int(t['args_words'][i]) != op.arity:
            return f"task {i}: {op.name} takes {op.arity} args, got {int(t['args_words'][i])}"
    ao, aw = t['args_off'].astype(np.int64), t['args_words'].astype(np.int64)
    if ((ao < 0) | (ao + aw > len(b.args))).any():
        return f'task {int(np.argmax((ao < 0) | (ao + aw > len(b.args))))}: args range'
    so, sc = t['succ_off'].astype(np.int64), t['succ_cnt'].astype(np.int64)
    bad = (so < 0) | (sc < 0) | (so + sc > len(b.succ))
    if bad.any():
        return f'task {int(np.argmax(bad))}: successor range'
    bad = (t['priority'] < 0) | (t['priority'] >= abi.NUM_PRIORITIES)
    if bad.any():
        return f"task {int(np.argmax(bad))}: priority outside [0,{abi.NUM_PRIORITIES - 1}]"
    bad = t['deadline_us'] < -1
    if bad.any():
        return f'task {int(np.argmax(bad))}: deadline_us'
    for f in ('wait_var', 'pub_var'):
        bad = (t[f] < -1) | (t[f] >= nvars)
        if bad.any():
            return f'task {int(np.argmax(bad))}: version variable {int(t[f][np.argmax(bad)])} out of range'
    bad = ((t['wait_var'] >= 0) & (t['wait_ver'] < 0)) | ((t['pub_var'] >= 0) & (t['pub_ver'] < 1))
    if bad.any():
        return f'task {int(np.argmax(bad))}: wait_ver >= 0 and pub_ver >= 1 (0 is the initial state)'
    for i in range(nt):
        op = ops[int(t['op_id'][i])]
        for j, a in enumerate(op.args):
            if a.type == 'buf':
                w = int(b.args[ao[i] + j])
                if (w == -1 and not a.optional) or w < -1 or w >= nbufs:
                    return f'task {i}: {op.name} arg {j} buffer index {w} out of range'
    # the edges as the descriptors address them (succ_off / succ_cnt need not tile the successor array)
    total = int(sc.sum())
    owner = np.repeat(np.arange(nt), sc)
    eidx = np.repeat(so, sc) + (np.arange(total) - np.repeat(np.cumsum(sc) - sc, sc))
    edges = b.succ[eidx].astype(np.int64) if total else np.zeros(0, np.int64)
    bad = (edges < 0) | (edges >= nt) | (edges == owner)
    if bad.any():
        k = int(np.argmax(bad))
        return f'task {int(owner[k])}: successor {int(edges[k])} out of range'
    indeg = np.bincount(edges, minlength=nt)
    if (indeg != t['indegree']).any():
        i = int(np.argmax(indeg != t['indegree']))
        return f"task {i}: indegree {int(t['indegree'][i])} != in-edges {int(indeg[i])}"
    rem, done = indeg.copy(), 0
    frontier = np.flatnonzero(rem == 0)
    first = np.cumsum(sc) - sc
    while len(frontier):
        done += len(frontier)
        idx = np.concatenate([np.arange(first[u], first[u] + sc[u]) for u in frontier]) if len(frontier) < 64 else \
            np.flatnonzero(np.isin(owner, frontier))
        s = edges[idx.astype(np.int64)]
        np.subtract.at(rem, s, 1)
        frontier = np.unique(s[rem[s] == 0])
    if done != nt:
        return 'dependency cycle'
    return ''


def pack_bundle(final_tasks, preds, buffers, variables, publishers, reads, final_version):
    """Pack tasks (dicts with op, words, priority, deadline_us, wait, pub, gi, name) and predecessor lists into the
    descriptor / successor / argument arrays plus metadata.json's content (`runtime/compile_workload.py:654-685`)."""
    ops = abi.load_ops()
    nt = len(final_tasks)
    indeg = np.array([len(p) for p in preds], dtype=np.int32)
    src = np.fromiter((p for ps in preds for p in ps), dtype=np.int64, count=int(indeg.sum()))
    dst = np.repeat(np.arange(nt, dtype=np.int64), indeg)
    order = np.argsort(src, kind='stable')
    succ = dst[order].astype('<i4')
    succ_cnt = np.bincount(src, minlength=nt).astype(np.int32)
    succ_off = np.concatenate([[0], np.cumsum(succ_cnt)[:-1]]).astype(np.int32)
    tasks = np.zeros(nt, dtype=abi.TASK_DTYPE)
    nwords = np.array([len(t['words']) for t in final_tasks], dtype=np.int32)
    tasks['op_id'] = [t['op'].id for t in final_tasks]
    tasks['succ_off'], tasks['succ_cnt'], tasks['indegree'] = succ_off, succ_cnt, indeg
    tasks['priority'] = [t['priority'] for t in final_tasks]
    tasks['deadline_us'] = [t.get('deadline_us', -1) for t in final_tasks]
    tasks['args_off'] = np.concatenate([[0], np.cumsum(nwords)[:-1]])
    tasks['args_words'] = nwords
    tasks['wait_var'], tasks['pub_var'] = abi.NO_VAR, abi.NO_VAR
    tasks['workload_id'] = [t.get('gi', 0) for t in final_tasks]
    for i, t in enumerate(final_tasks):
        if t.get('wait'):
            tasks['wait_var'][i], tasks['wait_ver'][i] = variables[t['wait'][0]]['id'], t['wait'][1]
        if t.get('pub'):
            tasks['pub_var'][i], tasks['pub_ver'][i] = variables[t['pub'][0]]['id'], t['pub'][1]
    args = np.fromiter((w for t in final_tasks for w in t['words']), dtype='<i4', count=int(nwords.sum()))
    meta = {
        'abi_version': abi.ABI_VERSION, 'task_count': nt, 'edge_count': int(len(succ)), 'args_words': int(len(args)),
        'task_names': [t['name'] for t in final_tasks],
        'initial_ready': [int(i) for i in np.flatnonzero(indeg == 0)],
        'operator_ids': {o.name: o.id for o in ops.values()},
        'buffers': buffers,
        'variables': list(variables.values()),
        'publishers': publishers,
        'reads': reads,
        'final_versions': final_version,
    }
    return tasks, succ, args, meta


# ------------------------------------------------------------------------------------------------ JSON -> bundle

def _bf16_value(x: float) -> float:
    if x != x or math.isinf(x):
        return x
    bits = int(np.array([x], '<f4').view('<u4')[0])
    return float(np.array([(bits + 0x7FFF + ((bits >> 16) & 1)) & 0xFFFF0000], '<u4').view('<f4')[0])


def _parse_init(where, init, rows, cols, dtype):
    _need(isinstance(init, dict) and 'kind' in init, f"{where}: init must be an object with a 'kind'")
    kind, n = init['kind'], rows * cols
    if dtype == 'i32':
        conv = int
    elif dtype == 'bf16':
        conv = lambda x: _bf16_value(float(np.float32(x)))
    else:
        conv = lambda x: float(np.float32(x))
    if kind == 'fill':
        return {'kind': 'fill', 'value': conv(init['value'])}
    if kind == 'values':
        raw = init['values']
        _need(isinstance(raw, list) and len(raw) == n, f'{where}: init.values must be a list of {n} numbers')
        return {'kind': 'values', 'values': [conv(x) for x in raw]}
    if kind == 'seeded':
        # the reference compiler takes seeded only for f32; here a bf16 buffer may be seeded too (value rounded once to bf16):
        # serving weights of the 8B-shape decode workload are generated in place instead of through 30 GB of f32 masters
        _need(dtype in ('f32', 'bf16'), f'{where}: seeded init needs dtype f32 or bf16')
        scale = float(np.float32(init['scale']))
        dist = init.get('dist', 'normal')
        draws, bias, coef = seeded_params(dist, scale)
        return {'kind': 'seeded', 'seed': int(init['seed']), 'scale': scale, 'dist': dist, 'draws': draws, 'bias': bias, 'coef': coef}
    if kind == 'file':
        p = Path(init['path'])
        _need(not p.is_absolute() and '..' not in p.parts, f'{where}: init.path must be relative to the bundle')
        return {'kind': 'file', 'path': p.as_posix()}
    raise CompileError(f"{where}: init.kind must be one of 'fill', 'values', 'seeded', 'file', got {kind!r}")


def compile_spec(spec: dict, base_versions: dict | None = None, data_dir=None, blobs: dict | None = None) -> Bundle:
    """Workload JSON (already parsed) -> Bundle."""
    ops = abi.load_ops()
    _need(isinstance(spec, dict) and 'graphs' in spec, "workload: expected an object with 'graphs'")
    base_versions = dict(base_versions or {})
    var_names = spec.get('variables', [])
    _need(len(set(var_names)) == len(var_names), 'workload: duplicate variable names')
    variables = {n: {'name': n, 'id': i, 'base_version': int(base_versions.get(n, 0))} for i, n in enumerate(var_names)}
    final_version = {n: v['base_version'] for n, v in variables.items()}

    buffers, buf_index = [], {}
    for i, d in enumerate(spec.get('buffers', [])):
        name = d['name']
        _need(name not in buf_index, f'buffers[{i}]: duplicate buffer {name!r}')
        rows, cols, dtype = int(d.get('rows', 1)), int(d.get('cols', 1)), d.get('dtype', 'f32')
        _need(rows >= 1 and cols >= 1 and rows * cols <= INT32_MAX, f'buffer {name!r}: bad shape {rows}x{cols}')
        _need(dtype in abi.DTYPES, f'buffer {name!r}: dtype must be one of {sorted(abi.DTYPES)}')
        init = _parse_init(f'buffer {name!r}', d.get('init', {'kind': 'fill', 'value': 0}), rows, cols, dtype)
        buf_index[name] = len(buffers)
        buffers.append({'name': name, 'index': len(buffers), 'rows': rows, 'cols': cols, 'dtype': abi.DTYPES[dtype], 'init': init})

    # ---- declared tasks
    decls, index_of = [], {}
    for gi, g in enumerate(spec['graphs']):
        gname = g.get('name', f'g{gi}')
        for ti, t in enumerate(g['tasks']):
            where = f"{gname}/{t['id']}"
            _need(where not in index_of, f'{where}: duplicate task id')
            op = ops.get(t['op'])
            _need(op is not None, f"{where}: unknown op {t['op']!r}")
            given = t.get('args', {})
            _need(set(given) <= {a.name for a in op.args}, f'{where}: unknown argument(s) {sorted(set(given) - {a.name for a in op.args})}')
            words = []
            for a in op.args:
                v = given.get(a.name)
                if a.type == 'buf':
                    if v is None:
                        _need(a.optional, f'{where}: required buffer argument {a.name!r} missing')
                        words.append(abi.ABSENT_BUF)
                    else:
                        _need(v in buf_index, f'{where}: argument {a.name!r} names undeclared buffer {v!r}')
                        words.append(buf_index[v])
                elif a.type == 'i32':
                    _need(v is not None and int(v) == v and -2**31 <= v <= INT32_MAX, f'{where}: argument {a.name!r} must be an int32')
                    words.append(int(v))
                else:
                    _need(v is not None, f'{where}: argument {a.name!r} missing')
                    words.append(abi.f32_word(float(v)))
            prio = int(t.get('priority', 0))
            _need(0 <= prio < abi.NUM_PRIORITIES, f'{where}: priority {prio} outside [0,{abi.NUM_PRIORITIES - 1}]')
            index_of[where] = len(decls)
            decls.append({'name': where, 'graph': gname, 'gi': gi, 'op': op, 'words': words, 'priority': prio,
                          'deadline_us': int(t.get('deadline_us', -1)), 'after': t.get('after', []),
                          'publishes': t.get('publishes'), 'reads': t.get('reads', []), 'pub': None, 'wait': None, 'gate': False})
    for d in decls:
        deps = []
        for a in d['after']:
            key = f"{d['graph']}/{a}" if f"{d['graph']}/{a}" in index_of else a
            _need(key in index_of, f"{d['name']}: 'after' names unknown task {a!r}")
            deps.append(index_of[key])
        d['deps'] = deps

    # ---- versions
    publishers = {n: [] for n in variables}
    for i, d in enumerate(decls):
        if d['publishes'] is not None:
            _need(d['publishes'] in variables, f"{d['name']}: publishes undeclared variable {d['publishes']!r}")
            final_version[d['publishes']] += 1
            publishers[d['publishes']].append(i)
            d['pub'] = (d['publishes'], final_version[d['publishes']])
    by_version = {v: {variables[v]['base_version'] + k + 1: i for k, i in enumerate(idx)} for v, idx in publishers.items()}
    exact_edges, reads_meta = [], []
    for i, d in enumerate(decls):
        waits = []
        for r in d['reads']:
            var, policy, n = r['var'], r.get('policy', 'at_least'), int(r['version'])
            _need(var in variables, f"{d['name']}: reads undeclared variable {var!r}")
            _need(policy in ('exact', 'at_least'), f"{d['name']}: read policy must be exact or at_least")
            base = variables[var]['base_version']
            if policy == 'exact':
                _need(n >= base, f"{d['name']}: exact read of {var!r} at version {n} is stale (base_version={base})")
            if n > base:
                _need(n in by_version[var], f"{d['name']}: read of {var!r} at version {n} can never be satisfied")
            nxt = by_version[var].get(n + 1)
            if policy == 'exact' and nxt is not None and nxt != i:
                exact_edges.append((i, nxt))
            if n > 0:
                waits.append((var, n))
            reads_meta.append({'task': i, 'var': var, 'policy': policy, 'version': n})
        d['waits'] = waits
    for var, idx in publishers.items():
        base = variables[var]['base_version']
        if idx and base > 0:
            d = decls[idx[0]]
            own = [k for k, (v, _) in enumerate(d['waits']) if v == var]
            if own:
                d['waits'][own[0]] = (var, max(d['waits'][own[0]][1], base))
            else:
                d['waits'].append((var, base))

    # ---- layout with gates
    final_tasks, final_of, gates_of = [], [0] * len(decls), {}
    noop = ops['noop']
    for i, d in enumerate(decls):
        for k, (var, ver) in enumerate(d['waits'][1:], 1):
            gates_of.setdefault(i, []).append(len(final_tasks))
            final_tasks.append({'name': f"__gate/{d['name']}/{k}", 'gi': d['gi'], 'op': noop, 'words': [], 'priority': d['priority'],
                                'deadline_us': d['deadline_us'], 'pub': None, 'wait': (var, ver), 'gate': True})
        final_of[i] = len(final_tasks)
        if d['waits']:
            d['wait'] = d['waits'][0]
        final_tasks.append(d)
    nt = len(final_tasks)
    preds = [[] for _ in range(nt)]
    for i, d in enumerate(decls):
        preds[final_of[i]] = gates_of.get(i, []) + sorted({final_of[j] for j in d['deps']})
    for reader, nxt in exact_edges:
        if final_of[reader] not in preds[final_of[nxt]]:
            preds[final_of[nxt]].append(final_of[reader])

    pub_list = [{'task': final_of[i], 'name': decls[i]['name'], 'var': variables[v]['id'], 'version': decls[i]['pub'][1]}
                for v, idx in publishers.items() for i in idx]
    tasks, succ, args, meta = pack_bundle(final_tasks, preds, buffers, variables, pub_list,
                                          [{**r, 'task': final_of[r['task']]} for r in reads_meta], final_version)
    b = Bundle(tasks, succ, args, meta, Path(data_dir) if data_dir else None, dict(blobs or {}))
    problem = validate(b)
    _need(not problem, f'compiled bundle is malformed: {problem}')
    return b
