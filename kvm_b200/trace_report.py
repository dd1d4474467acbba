"""Where the time of one launch goes, from the executor's per-task trace (start / end %globaltimer and SM per task).

    python -m kvm_b200.trace_report train  [gpt_162m]      per-op table and a utilisation timeline of one training step
    python -m kvm_b200.trace_report decode [qwen3_8b_4l]   per-phase table of one decode token, with the streamed tasks' detail

Busy fraction = sum(end - start) / (workers x span), the reference's formula
(results/2026-11-11-162m-ceiling/README.md:50-56).  Tracing adds two timestamps and a store per task.
"""
import collections
import re
import sys

import numpy as np

from . import abi
from .executor import Executor


def _traced(bundle, warm=3):
    ex = Executor(trace=True)
    ex.load(bundle)
    for _ in range(warm):
        ex.run()
    res = ex.run()
    st, en, sm = ex.trace()
    det = ex.trace_detail() if ex.plan_info()[0] else np.zeros(len(st), np.int32)
    info = (ex.launch_info()[0], ex.plan_info())
    ex.close()
    return res, st.astype(np.float64), en.astype(np.float64), sm, det, info


def train(model='gpt_162m', windows=60):
    from .workloads.gpt import build_training, preset
    cfg = preset(model)
    bundle = build_training(cfg, 1, stream_steps=16).to_bundle(check=False)
    names = {v.id: k for k, v in abi.load_ops().items()}
    res, st, en, _, _, (workers, _) = _traced(bundle)
    ok = (en > st) & (st > 0)
    t0, span = st[ok].min(), en[ok].max() - st[ok].min()
    dur = (en - st) * ok
    opid = bundle.tasks['op_id']
    print(f'{model}: {len(bundle.tasks)} tasks, {res.ms:.3f} ms by CUDA events, span {span / 1e6:.3f} ms, {workers} workers, busy {dur.sum() / (workers * span):.3f}')
    print(f'{"op":24s} {"tasks":>7s} {"SM-time ms":>11s} {"share":>6s} {"mean us":>8s}')
    rows = []
    for op in np.unique(opid):
        sel = opid == op
        rows.append((dur[sel].sum(), names.get(int(op), str(op)), int(sel.sum()), dur[sel].mean()))
    for tot, name, n, mean in sorted(rows, reverse=True):
        print(f'{name:24s} {n:7d} {tot / 1e6 / workers:11.3f} {tot / (workers * span):6.3f} {mean / 1e3:8.2f}')
    print(f'{"idle":24s} {"":7s} {(workers * span - dur.sum()) / 1e6 / workers:11.3f} {1 - dur.sum() / (workers * span):6.3f}')
    print(f'\ntimeline ({windows} windows): busy workers of {workers}, the three op kinds that hold most of them')
    edges = np.linspace(0, span, windows + 1)
    for w in range(windows):
        a, b = edges[w], edges[w + 1]
        d = (np.clip(en - t0, a, b) - np.clip(st - t0, a, b)) * ok
        fam = collections.Counter()
        for op in np.unique(opid[d > 0]):
            fam[names.get(int(op), str(op))] += d[opid == op].sum() / (b - a)
        print(f'{a / 1e6:6.2f}-{b / 1e6:6.2f} ms  {d.sum() / (b - a):6.1f}  ' + ', '.join(f'{k} {v:.0f}' for k, v in fam.most_common(3)))


PHASE = {'q': '1 qkv', 'k': '1 qkv', 'v': '1 qkv', 'part': '2 attention split', 'merge': '3 merge', 'o': '4 o', 'gate': '5 gate/up', 'up': '5 gate/up', 'down': '6 down'}


def decode(model='qwen3_8b_4l'):
    from .workloads.decode import build_decode, preset
    cfg = preset(model)
    bundle = build_decode(cfg).to_bundle(check=False)
    names = bundle.metadata['task_names']
    res, st, en, sm, det, (workers, plan) = _traced(bundle)
    t0 = st[st > 0].min()
    st, en = (st - t0) / 1e3, (en - t0) / 1e3
    print(f'{model}: {len(names)} tasks per token, {res.ms * 1e3:.1f} us by CUDA events, static {plan[0]}, stream ring {plan[1]}, busy {res.busy_frac:.3f}')
    groups = collections.OrderedDict()
    for i, n in enumerate(names):
        m = re.search(r'l(\d+)\.(q|k|v|part|merge|o|gate|up|down)\b', n)
        key = (int(m.group(1)), PHASE[m.group(2)]) if m else (1 << 20, re.sub(r'\d+', '#', n.split('/')[-1]))
        groups.setdefault(key, []).append(i)
    print(f'{"layer":>5s} {"phase":18s} {"tasks":>5s} {"first start":>11s} {"last end":>9s} {"gap":>5s} {"mean":>6s} | streamed tasks: prologue, stage loop, of it waiting, rest (us)')
    prev_end = 0.0
    for key in sorted(groups):
        idx = np.array(groups[key])
        d = en[idx] - st[idx]
        line = f'{key[0] if key[0] < (1 << 20) else "":>5} {key[1]:18s} {len(idx):5d} {st[idx].min():11.1f} {en[idx].max():9.1f} {st[idx].min() - prev_end:5.1f} {d.mean():6.1f}'
        dd = det[idx]
        if (dd != 0).any():
            unit = 0.1 if 'attention' in key[1] else 0.2
            pro, loop, wait = (dd & 255) * unit, ((dd >> 8) & 255) * unit, ((dd >> 16) & 255) * 0.2
            if 'attention' in key[1]:
                line += f' | prologue {pro.mean():4.1f}, waits for keys and values {loop.mean():4.1f}, rest {(d - pro - loop).mean():4.1f}'
            else:
                line += f' | {pro.mean():4.1f}, {loop.mean():5.1f}, {wait.mean():4.1f}, {(d - pro - loop).mean():4.1f}'
        print(line)
        prev_end = en[idx].max()


if __name__ == '__main__':
    what = sys.argv[1] if len(sys.argv) > 1 else 'train'
    {'train': train, 'decode': decode}[what](*sys.argv[2:3])
