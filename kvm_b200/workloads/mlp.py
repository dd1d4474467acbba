"""Several independent MLP classifiers trained side by side in one task graph (one executor launch runs them all).

Each model: x[batch, in_dim] -> W1 -> ReLU -> W2 -> ReLU -> W3 -> softmax cross-entropy over `classes`, float32 storage,
SGD with momentum.  Everything is expressed with ops of the reference registry: matmul_tile (bias in the epilogue, the
pre-activation kept through `pre`), act_fwd / act_bwd (kind 0 = ReLU), softmax_ce_fused, colsum for the bias gradients, and
the momentum update composed as  v = mu*v (scale_flat);  v += g (residual_add);  w -= lr*v (sgd_range)
(include/mvm_ops_gpt.def, include/mvm_ops_extra.def:55-63 of the reference).  The models share the input batches and
nothing else, so the graph has one connected component per model and the executor interleaves them freely.
"""
from __future__ import annotations

import math
import zlib
from dataclasses import dataclass, replace

import numpy as np

from .graph import Graph


@dataclass(frozen=True)
class MLPConfig:
    name: str = 'mlp8'
    widths: tuple = (128, 256, 384, 512, 768, 1024, 1536, 2048)
    in_dim: int = 512
    classes: int = 10
    batch: int = 256
    lr: float = 1e-2
    momentum: float = 0.9
    seed: int = 0
    flat_chunk: int = 1 << 16     # elements per elementwise / optimizer task


PRESETS = {
    'mlp8': MLPConfig(),
    'mlp_small': MLPConfig(name='mlp_small', widths=(64, 128), in_dim=64, batch=64),
}


def preset(name, **over):
    return replace(PRESETS[name], **over)


def params(c: MLPConfig) -> int:
    return sum(c.in_dim * w + w + w * w + w + w * c.classes + c.classes for w in c.widths)


def build_mlps(c: MLPConfig, steps: int) -> Graph:
    g = Graph('mlp')
    B, D, C = c.batch, c.in_dim, c.classes
    seeded = lambda name, scale, dist: {'kind': 'seeded', 'seed': zlib.crc32(f'{c.seed}/{name}'.encode()), 'scale': scale, 'dist': dist}
    rng = np.random.default_rng(c.seed + 1)
    xs, ys = [], []
    for s in range(steps):                       # the batches are shared by the models
        xs.append(g.buffer(f'x.{s}', B, D, init=seeded(f'x.{s}', 1.0, 'normal')))
        ys.append(g.data(f'y.{s}', rng.integers(0, C, size=(B, 1), dtype=np.int32), 'i32'))

    def mm(tag, a, b, out, M, N, K, flags=0, bias=None, pre=None, prio=10):
        for m0 in range(0, M, 64):
            for n0 in range(0, N, 64):
                m1, n1 = min(m0 + 64, M), min(n0 + 64, N)
                ra = (a, (0, K), (m0, m1)) if flags & 1 else (a, (m0, m1), (0, K))
                rb = (b, (n0, n1), (0, K)) if flags & 2 else (b, (0, K), (n0, n1))
                g.task('matmul_tile', {'a': a, 'b': b, 'out': out, 'bias': bias, 'res': None, 'pre': pre, 'm0': m0, 'n0': n0, 'M': M, 'N': N, 'K': K,
                                       'flags': flags, 'alpha': 1.0},
                       [ra, rb, (bias, (0, 1), (n0, n1)) if bias else None], [(out, (m0, m1), (n0, n1)), (pre, (m0, m1), (n0, n1)) if pre else None],
                       prio, f'{tag}.{m0 // 64}.{n0 // 64}')

    def flat(op, tag, bufs, n, extra, reads, writes, prio=10):
        for i, (e0, e1) in enumerate(g.flat_chunks(writes[0], c.flat_chunk)):      # chunks on row boundaries: no false dependencies
            g.task(op, dict(bufs, e0=e0, e1=e1, **extra), [(b, *g.region_of(b, e0, e1)) for b in reads], [(b, *g.region_of(b, e0, e1)) for b in writes], prio, f'{tag}.{i}')

    for mi, w in enumerate(c.widths):
        p = f'm{mi}.'
        shapes = {'w1': (D, w), 'b1': (1, w), 'w2': (w, w), 'b2': (1, w), 'w3': (w, C), 'b3': (1, C)}
        for n, (r, cc) in shapes.items():
            fan_in = {'w1': D, 'w2': w, 'w3': w}.get(n)
            init = seeded(p + n, math.sqrt(6.0 / fan_in), 'uniform') if fan_in else {'kind': 'fill', 'value': 0.0}
            g.buffer(p + n, r, cc, init=init)
            g.buffer(p + 'g.' + n, r, cc)
            g.buffer(p + 'v.' + n, r, cc, init={'kind': 'fill', 'value': 0.0})
        for n, cc in (('h1pre', w), ('h1', w), ('h2pre', w), ('h2', w), ('dh2', w), ('dh1', w)):
            g.buffer(p + n, B, cc)
        g.buffer(p + 'logits', B, C), g.buffer(p + 'dlogits', B, C), g.buffer(p + 'rowloss', B, 1), g.buffer(p + 'lse', B, 1)
        for s in range(steps):
            x, y, t = xs[s], ys[s], f'{p}s{s}.'
            loss = g.buffer(f'{p}loss.{s}', 1, 2)
            mm(t + 'fc1', x, p + 'w1', p + 'h1pre', B, w, D, bias=p + 'b1')
            flat('act_fwd', t + 'relu1', {'x': p + 'h1pre', 'out': p + 'h1'}, B * w, {'kind': 0}, [p + 'h1pre'], [p + 'h1'])
            mm(t + 'fc2', p + 'h1', p + 'w2', p + 'h2pre', B, w, w, bias=p + 'b2')
            flat('act_fwd', t + 'relu2', {'x': p + 'h2pre', 'out': p + 'h2'}, B * w, {'kind': 0}, [p + 'h2pre'], [p + 'h2'])
            mm(t + 'fc3', p + 'h2', p + 'w3', p + 'logits', B, C, w, bias=p + 'b3')
            g.task('softmax_ce_fused', {'logits': p + 'logits', 'tgt': y, 'rowloss': p + 'rowloss', 'lse': p + 'lse', 'dlogits': p + 'dlogits', 'r0': 0, 'r1': B, 'V': C,
                                        'ignore': -1, 'N': B, 'scale': 1.0}, [p + 'logits', y], [p + 'rowloss', p + 'lse', p + 'dlogits'], 10, t + 'ce')
            g.task('softmax_ce_reduce', {'rowloss': p + 'rowloss', 'tgt': y, 'loss': loss, 'N': B, 'ignore': -1}, [p + 'rowloss', y], [loss], 1, t + 'loss')
            # backward
            mm(t + 'dw3', p + 'h2', p + 'dlogits', p + 'g.w3', w, C, B, flags=1)
            g.task('colsum', {'x': p + 'dlogits', 'out': p + 'g.b3', 'R': B, 'c0': 0, 'c1': C, 'acc': 0}, [p + 'dlogits'], [p + 'g.b3'], 5, t + 'db3')
            mm(t + 'dh2', p + 'dlogits', p + 'w3', p + 'dh2', B, w, C, flags=2)
            flat('act_bwd', t + 'drelu2', {'x': p + 'h2pre', 'dy': p + 'dh2', 'dx': p + 'dh2'}, B * w, {'kind': 0, 'acc': 0}, [p + 'h2pre', p + 'dh2'], [p + 'dh2'])
            mm(t + 'dw2', p + 'h1', p + 'dh2', p + 'g.w2', w, w, B, flags=1)
            for c0 in range(0, w, 256):
                g.task('colsum', {'x': p + 'dh2', 'out': p + 'g.b2', 'R': B, 'c0': c0, 'c1': min(c0 + 256, w), 'acc': 0},
                       [(p + 'dh2', (0, B), (c0, min(c0 + 256, w)))], [(p + 'g.b2', (0, 1), (c0, min(c0 + 256, w)))], 5, f'{t}db2.{c0 // 256}')
            mm(t + 'dh1', p + 'dh2', p + 'w2', p + 'dh1', B, w, w, flags=2)
            flat('act_bwd', t + 'drelu1', {'x': p + 'h1pre', 'dy': p + 'dh1', 'dx': p + 'dh1'}, B * w, {'kind': 0, 'acc': 0}, [p + 'h1pre', p + 'dh1'], [p + 'dh1'])
            mm(t + 'dw1', x, p + 'dh1', p + 'g.w1', D, w, B, flags=1)
            for c0 in range(0, w, 256):
                g.task('colsum', {'x': p + 'dh1', 'out': p + 'g.b1', 'R': B, 'c0': c0, 'c1': min(c0 + 256, w), 'acc': 0},
                       [(p + 'dh1', (0, B), (c0, min(c0 + 256, w)))], [(p + 'g.b1', (0, 1), (c0, min(c0 + 256, w)))], 5, f'{t}db1.{c0 // 256}')
            # SGD with momentum: v = mu v + g;  w -= lr v
            for n, (r, cc) in shapes.items():
                wn, gn, vn, ne = p + n, p + 'g.' + n, p + 'v.' + n, r * cc
                flat('scale_flat', f'{t}mu.{n}', {'x': vn, 'out': vn}, ne, {'alpha': c.momentum}, [vn], [vn], 3)
                flat('residual_add', f'{t}acc.{n}', {'a': vn, 'b': gn, 'out': vn}, ne, {}, [vn, gn], [vn], 3)
                flat('sgd_range', f'{t}sgd.{n}', {'w': wn, 'g': vn}, ne, {'lr': c.lr}, [wn, vn], [wn], 3)
    return g
