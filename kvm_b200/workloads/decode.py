"""Greedy decode workloads in the reference's task ABI: a Llama/Qwen-shaped decoder (RMSNorm, GQA with RoPE, SwiGLU) generating
one token per run for `batch` independent users, one row per user as the reference serves (`frontend/mvmfe/serve.py:1-11,72-83`).

Per layer and user: q/k/v = gemv_bf16 with the RMSNorm prologue (pro 1); attn_decode_part over S context splits with fused
RoPE + KV append (flags 3) and attn_decode_merge; o-projection gemv with the residual; gate / up gemv (pro 1); down-projection
gemv with the SwiGLU prologue (pro 2) and the residual.  Then final norm folded into the LM-head gemv, argmax, and the
bookkeeping for the next token (token -> gather_rows of the embedding, lens += 1).  Re-arming the one-token template generates
the next token.  Op semantics: include/mvm_ops_extra.def:79-95 of the reference.  Weights are bf16 [N, K] serving copies
(`serve.py:317-344`), here seeded in place; the KV cache is prefilled with seeded values standing in for a prompt of `ctx` tokens.
QK RMSNorm (Qwen3) is not part of the reference op set: `qk_norm=True` uses this executor's extension op attn_decode_part_qkn
(id 300, include/kvm_ops.def), which is attn_decode_part with the per-head normalisation in front of the rotary embedding.
"""
from __future__ import annotations

import zlib
from dataclasses import dataclass, replace

import numpy as np

from .graph import Graph


@dataclass(frozen=True)
class DecodeConfig:
    name: str = 'decode_tiny'
    layers: int = 2
    hidden: int = 256
    heads: int = 8
    kv_heads: int = 2
    head_dim: int = 32
    ffn: int = 512
    vocab: int = 1000
    ctx: int = 40            # tokens already in the cache
    tmax: int = 128
    batch: int = 1
    splits: int = 4
    theta: float = 1e6
    eps: float = 1e-6
    init_std: float = 0.02
    seed: int = 0
    rows_per_task: int = 64  # weight rows per gemv task; 0 = balance every phase over `workers` SMs
    workers: int = 148
    join_threshold: int = 24  # fan-ins wider than this go through a join no-op (fewer edges, one more hop)
    lockstep: bool = False    # several users: keep them in step phase by phase (see build_decode); measured slower, kept for experiments
    qk_norm: bool = False     # Qwen3: RMSNorm of every query head and of the new key over the head dimension before RoPE (extension op attn_decode_part_qkn)


PRESETS = {
    'decode_tiny': DecodeConfig(),
    # BASELINE config 5 (Qwen3-8B shape), 4K context.  17 context splits: a split's keys (at most 256 of 128 bf16 values) fit one 64 KB
    # stage of the stream ring, and 8 kv heads x 17 splits = 136 tasks are one wave over the SMs
    'qwen3_8b': DecodeConfig(name='qwen3_8b', layers=36, hidden=4096, heads=32, kv_heads=8, head_dim=128, ffn=12288, vocab=151936, ctx=4096, tmax=4096 + 256,
                             splits=17, rows_per_task=0, join_threshold=1000),
    'qwen3_8b_4l': DecodeConfig(name='qwen3_8b_4l', layers=4, hidden=4096, heads=32, kv_heads=8, head_dim=128, ffn=12288, vocab=151936, ctx=4096, tmax=4096 + 256,
                                splits=17, rows_per_task=0, join_threshold=1000),
}


def preset(name, **over):
    return replace(PRESETS[name], **over)


def weight_bytes(c: DecodeConfig) -> int:
    """bf16 bytes one token reads: all projection weights + LM head (the embedding row is negligible)."""
    per_layer = c.hidden * (c.heads + 2 * c.kv_heads) * c.head_dim + c.heads * c.head_dim * c.hidden + 3 * c.hidden * c.ffn
    return 2 * (c.layers * per_layer + c.vocab * c.hidden)


def kv_bytes(c: DecodeConfig, ctx: int) -> int:
    return c.layers * 2 * c.kv_heads * ctx * c.head_dim * 2


def build_decode(c: DecodeConfig) -> Graph:
    g = Graph('decode')
    g.join_threshold = c.join_threshold
    d, H, Hkv, hd, F, V, B, S = c.hidden, c.heads, c.kv_heads, c.head_dim, c.ffn, c.vocab, c.batch, c.splits
    seeded = lambda name, scale=None: {'kind': 'seeded', 'seed': zlib.crc32(f'{c.seed}/{name}'.encode()), 'scale': scale or c.init_std, 'dist': 'normal'}

    def W(name, n, k):
        return g.buffer('wb.' + name, n, k, 'bf16', seeded(name))

    def phase_rows(ns, k):
        """Weight rows per task for a phase of concurrent GEMVs with ns[i] rows of length k: the smallest equal share that fits
        the phase into whole waves over the SMs, with as many waves as keep a task near 2 MB of weights."""
        if c.rows_per_task > 0:
            return c.rows_per_task
        total = sum(ns) * B                      # every user streams the rows again
        slots = c.workers * max(1, round(total * k * 2 / (c.workers * (2 << 20))))
        rows = max(8, -(-total // slots))
        while sum(-(-n // rows) for n in ns) * B > slots:
            rows += 1
        return rows

    g.buffer('wb.embed', V, d, 'bf16', seeded('embed'))
    g.buffer('w.lnf', 1, d, init={'kind': 'fill', 'value': 1.0})
    W('head', V, d)
    for l in range(c.layers):
        p = f'l{l}.'
        g.buffer('w.' + p + 'ln1', 1, d, init={'kind': 'fill', 'value': 1.0}), g.buffer('w.' + p + 'ln2', 1, d, init={'kind': 'fill', 'value': 1.0})
        W(p + 'q', H * hd, d), W(p + 'k', Hkv * hd, d), W(p + 'v', Hkv * hd, d), W(p + 'o', d, H * hd), W(p + 'gate', F, d), W(p + 'up', F, d), W(p + 'down', d, F)
    # Every user is an independent one-row request with its own cache, length counter and activations (b = 0 in every op);
    # the weights are shared.  Emission is layer by layer and, inside a GEMV, weight-row block by block with the users innermost:
    # the users' tasks on one block of rows sit side by side in the ready queue, run at the same time on different SMs, and the
    # block comes from HBM once and from L2 for the others.
    U = range(B)
    T = [f'u{u}.' for u in U]
    lens = [g.buffer(T[u] + 'lens', 1, 1, 'i32', {'kind': 'fill', 'value': c.ctx}) for u in U]
    tok = [g.buffer(T[u] + 'tok', 1, 1, 'i32', {'kind': 'fill', 'value': (7 * u + 3) % V}) for u in U]
    x = [g.buffer(T[u] + 'x', 1, d) for u in U]
    for u in U:
        g.task('gather_rows', {'src': 'wb.embed', 'idx': tok[u], 'dst': x[u], 'r0': 0, 'r1': 1, 'd': d}, ['wb.embed', tok[u]], [x[u]], 31, T[u] + 'embed')

    def gemv_all(tag, xs, w, outs, n, k, pro=0, x2s=None, gamma=None, ress=None, prio=20, rows=None, after=()):
        rows = rows or phase_rows([n], k)
        for i, n0 in enumerate(range(0, n, rows)):
            n1 = min(n0 + rows, n)
            for u in U:
                x2, res = (x2s[u] if x2s else None), (ress[u] if ress else None)
                g.task('gemv_bf16', {'x': xs[u], 'x2': x2, 'gamma': gamma, 'w': w, 'out': outs[u], 'res': res, 'n0': n0, 'n1': n1, 'K': k, 'pro': pro, 'eps': c.eps},
                       [xs[u], x2, gamma, (w, (n0, n1)), (res, (0, 1), (n0, n1)) if res else None], [(outs[u], (0, 1), (n0, n1))], prio, f'{T[u]}{tag}.{i}', after=after)

    def lockstep(tag, bufs, prio):
        """With several users: a no-op that waits for every user's `bufs`; the next phase's tasks are released behind it in one
        go, block by block with the users side by side (that order is what lets the users share one HBM read of a block)."""
        if B == 1 or not c.lockstep:
            return ()
        return (g.task('noop', {}, list(bufs), [], prio, 'sync.' + tag),)

    G = H // Hkv
    bar = ()
    for l in range(c.layers):
        p = f'l{l}.'
        prio = max(30 - l, 2)
        TL = [f'{T[u]}l{l}.' for u in U]
        kc = [g.buffer(TL[u] + 'kc', Hkv * c.tmax, hd, 'bf16', seeded(TL[u] + 'kc', 1.0)) for u in U]
        vc = [g.buffer(TL[u] + 'vc', Hkv * c.tmax, hd, 'bf16', seeded(TL[u] + 'vc', 1.0)) for u in U]
        q, k, v = ([g.buffer(TL[u] + n, 1, cols) for u in U] for n, cols in (('q', H * hd), ('k', Hkv * hd), ('v', Hkv * hd)))
        r_qkv = phase_rows([H * hd, Hkv * hd, Hkv * hd], d)           # q, k and v run as one phase
        gemv_all(p + 'q', x, 'wb.' + p + 'q', q, H * hd, d, 1, gamma='w.' + p + 'ln1', prio=prio, rows=r_qkv, after=bar)
        gemv_all(p + 'k', x, 'wb.' + p + 'k', k, Hkv * hd, d, 1, gamma='w.' + p + 'ln1', prio=prio, rows=r_qkv, after=bar)
        gemv_all(p + 'v', x, 'wb.' + p + 'v', v, Hkv * hd, d, 1, gamma='w.' + p + 'ln1', prio=prio, rows=r_qkv, after=bar)
        part = [g.buffer(TL[u] + 'part', S * H, hd + 2) for u in U]
        o = [g.buffer(TL[u] + 'o', 1, H * hd) for u in U]
        slice_ = c.tmax // S
        qkn = None
        if c.qk_norm:        # per-layer weights of the two norms, rows (query, key), around one
            rng = np.random.default_rng(zlib.crc32(f'{c.seed}/{p}qkn'.encode()))
            qkn = g.data('w.' + p + 'qkn', (1.0 + 0.25 * rng.uniform(-1, 1, (2, hd))).astype(np.float32))
        for u in U:
            for kvh in range(Hkv):
                # Only the split that holds the newest key appends (one cache row); which one depends on the length at run time.
                # The splits of one step never touch each other's rows, so each declares a disjoint slice of the head's rows as
                # written (ordering against the next step comes through `lens`), and the S splits run concurrently.
                for s in range(S):
                    rows = (kvh * c.tmax + s * slice_, kvh * c.tmax + (s + 1) * slice_)
                    args = {'q': q[u], 'kc': kc[u], 'vc': vc[u], 'lens': lens[u], 'part': part[u], 'knew': k[u], 'vnew': v[u], 'b': 0, 'kvh': kvh, 's': s,
                            'S': S, 'H': H, 'Hkv': Hkv, 'hd': hd, 'Tmax': c.tmax, 'scale': hd ** -0.5, 'theta': c.theta, 'flags': 3}
                    if qkn:
                        args.update(qk_gamma=qkn, eps=c.eps)
                    g.task('attn_decode_part_qkn' if qkn else 'attn_decode_part', args,
                           [q[u], k[u], v[u], lens[u], qkn], [(kc[u], rows), (vc[u], rows), (part[u], (s * H + kvh * G, s * H + (kvh + 1) * G))], prio, f'{TL[u]}part.{kvh}.{s}')
        for u in U:
            for kvh in range(Hkv):                              # one merge per GQA group: short tasks, all concurrent
                g.task('attn_decode_merge', {'part': part[u], 'o': o[u], 'b': 0, 'h0': kvh * G, 'h1': (kvh + 1) * G, 'S': S, 'H': H, 'hd': hd},
                       [part[u]], [(o[u], (0, 1), (kvh * G * hd, (kvh + 1) * G * hd))], prio, f'{TL[u]}merge.{kvh}')
        x1 = [g.buffer(TL[u] + 'x1', 1, d) for u in U]
        bar = lockstep(p + 'o', o, prio)
        gemv_all(p + 'o', o, 'wb.' + p + 'o', x1, d, H * hd, 0, ress=x, prio=prio, after=bar)
        gate, up = ([g.buffer(TL[u] + n, 1, F) for u in U] for n in ('gate', 'up'))
        r_gu = phase_rows([F, F], d)
        bar = lockstep(p + 'gu', x1, prio)
        gemv_all(p + 'gate', x1, 'wb.' + p + 'gate', gate, F, d, 1, gamma='w.' + p + 'ln2', prio=prio, rows=r_gu, after=bar)
        gemv_all(p + 'up', x1, 'wb.' + p + 'up', up, F, d, 1, gamma='w.' + p + 'ln2', prio=prio, rows=r_gu, after=bar)
        xn = [g.buffer(TL[u] + 'x2', 1, d) for u in U]
        bar = lockstep(p + 'down', gate + up, prio)
        gemv_all(p + 'down', gate, 'wb.' + p + 'down', xn, d, F, 2, x2s=up, ress=x1, prio=prio, after=bar)
        x = xn
        bar = lockstep(p + 'next', x, prio)
    logits = [g.buffer(T[u] + 'logits', 1, V) for u in U]
    gemv_all('head', x, 'wb.head', logits, V, d, 1, gamma='w.lnf', prio=1, after=bar)
    for u in U:
        g.task('argmax', {'logits': logits[u], 'out': tok[u], 'r0': 0, 'r1': 1, 'V': V}, [logits[u]], [tok[u]], 1, T[u] + 'argmax')
        g.task('counter_inc', {'x': lens[u], 'i0': 0, 'i1': 1, 'delta': 1}, [lens[u]], [lens[u]], 0, T[u] + 'advance')
    return g


def build_decode_rows(c: DecodeConfig, exact_caches: bool = False) -> Graph:
    """The same decode step with the batch as ROWS of shared activation matrices (x [B, hidden], q [B, H*hd], ...), so that every
    projection is one pass over its weights for all users: gemv_bf16_rows (extension op 301) instead of one gemv_bf16 per user.
    Attention stays per user (each has its own cache rows and length; the ops take the user as their `b` argument), as do the
    split merges; embedding, argmax and the length counters run over the B rows at once.  Same weights (same seeds) as
    build_decode, so the tokens of user u equal those of build_decode's user u: exact_caches=True also gives every user the
    cache contents build_decode seeds for it (small configurations, parity tests); otherwise the combined caches are seeded."""
    from .. import initgen
    g = Graph('decode_rows')
    g.join_threshold = c.join_threshold
    d, H, Hkv, hd, F, V, B, S = c.hidden, c.heads, c.kv_heads, c.head_dim, c.ffn, c.vocab, c.batch, c.splits
    seed_of = lambda name: zlib.crc32(f'{c.seed}/{name}'.encode())
    seeded = lambda name, scale=None: {'kind': 'seeded', 'seed': seed_of(name), 'scale': scale or c.init_std, 'dist': 'normal'}
    W = lambda name, n, k: g.buffer('wb.' + name, n, k, 'bf16', seeded(name))

    def phase_rows(ns, k):
        if c.rows_per_task > 0:
            return c.rows_per_task
        total = sum(ns)
        slots = c.workers * max(1, round(total * k * 2 / (c.workers * (2 << 20))))
        rows = max(8, -(-total // slots))
        while sum(-(-n // rows) for n in ns) > slots:
            rows += 1
        # whole groups of eight weight rows (what one stage of the stream ring holds), at most seven of them: the static path's
        # tensor-core consumer keeps the partial sums of a task's row groups for all B activation rows in shared memory
        return min(-(-rows // 8) * 8, 56)

    def gemv(tag, x, w, out, n, k, pro=0, x2=None, gamma=None, res=None, prio=20, rows=None):
        rows = rows or phase_rows([n], k)
        for i, n0 in enumerate(range(0, n, rows)):
            n1 = min(n0 + rows, n)
            g.task('gemv_bf16_rows', {'x': x, 'x2': x2, 'gamma': gamma, 'w': w, 'out': out, 'res': res, 'n0': n0, 'n1': n1, 'K': k, 'pro': pro, 'eps': c.eps, 'r0': 0, 'r1': B},
                   [x, x2, gamma, (w, (n0, n1)), (res, (0, B), (n0, n1)) if res else None], [(out, (0, B), (n0, n1))], prio, f'{tag}.{i}')

    g.buffer('wb.embed', V, d, 'bf16', seeded('embed'))
    g.buffer('w.lnf', 1, d, init={'kind': 'fill', 'value': 1.0})
    W('head', V, d)
    for l in range(c.layers):
        p = f'l{l}.'
        g.buffer('w.' + p + 'ln1', 1, d, init={'kind': 'fill', 'value': 1.0}), g.buffer('w.' + p + 'ln2', 1, d, init={'kind': 'fill', 'value': 1.0})
        W(p + 'q', H * hd, d), W(p + 'k', Hkv * hd, d), W(p + 'v', Hkv * hd, d), W(p + 'o', d, H * hd), W(p + 'gate', F, d), W(p + 'up', F, d), W(p + 'down', d, F)
    lens = g.buffer('lens', B, 1, 'i32', {'kind': 'fill', 'value': c.ctx})
    tok = g.data('tok', np.array([[(7 * u + 3) % V] for u in range(B)], np.int32), 'i32')
    x = g.buffer('x', B, d)
    g.task('gather_rows', {'src': 'wb.embed', 'idx': tok, 'dst': x, 'r0': 0, 'r1': B, 'd': d}, ['wb.embed', tok], [x], 31, 'embed')
    G = H // Hkv
    slice_ = c.tmax // S
    for l in range(c.layers):
        p = f'l{l}.'
        prio = max(30 - l, 2)

        def cache(n):
            if exact_caches:
                draws, bias, coef = initgen.seeded_params('normal', 1.0)
                parts = [initgen.seeded_values(seed_of(f'u{u}.l{l}.{n}'), Hkv * c.tmax * hd, draws, bias, coef).reshape(Hkv * c.tmax, hd) for u in range(B)]
                return g.data(p + n, np.concatenate(parts), 'bf16')
            return g.buffer(p + n, B * Hkv * c.tmax, hd, 'bf16', seeded(p + n, 1.0))
        kc, vc = cache('kc'), cache('vc')
        q, k, v = (g.buffer(p + n, B, cols) for n, cols in (('q', H * hd), ('k', Hkv * hd), ('v', Hkv * hd)))
        r_qkv = phase_rows([H * hd, Hkv * hd, Hkv * hd], d)
        gemv(p + 'q', x, 'wb.' + p + 'q', q, H * hd, d, 1, gamma='w.' + p + 'ln1', prio=prio, rows=r_qkv)
        gemv(p + 'k', x, 'wb.' + p + 'k', k, Hkv * hd, d, 1, gamma='w.' + p + 'ln1', prio=prio, rows=r_qkv)
        gemv(p + 'v', x, 'wb.' + p + 'v', v, Hkv * hd, d, 1, gamma='w.' + p + 'ln1', prio=prio, rows=r_qkv)
        part, o = g.buffer(p + 'part', B * S * H, hd + 2), g.buffer(p + 'o', B, H * hd)
        qkn = None
        if c.qk_norm:
            rng = np.random.default_rng(zlib.crc32(f'{c.seed}/{p}qkn'.encode()))
            qkn = g.data('w.' + p + 'qkn', (1.0 + 0.25 * rng.uniform(-1, 1, (2, hd))).astype(np.float32))
        for u in range(B):
            for kvh in range(Hkv):
                base = (u * Hkv + kvh) * c.tmax
                for s in range(S):
                    rows = (base + s * slice_, base + (s + 1) * slice_)
                    args = {'q': q, 'kc': kc, 'vc': vc, 'lens': lens, 'part': part, 'knew': k, 'vnew': v, 'b': u, 'kvh': kvh, 's': s, 'S': S, 'H': H, 'Hkv': Hkv, 'hd': hd,
                            'Tmax': c.tmax, 'scale': hd ** -0.5, 'theta': c.theta, 'flags': 3}
                    if qkn:
                        args.update(qk_gamma=qkn, eps=c.eps)
                    prow = (u * S + s) * H + kvh * G
                    g.task('attn_decode_part_qkn' if qkn else 'attn_decode_part', args, [(q, (u, u + 1)), (k, (u, u + 1)), (v, (u, u + 1)), lens, qkn],
                           [(kc, rows), (vc, rows), (part, (prow, prow + G))], prio, f'{p}part.{u}.{kvh}.{s}')
        for u in range(B):
            for kvh in range(Hkv):
                g.task('attn_decode_merge', {'part': part, 'o': o, 'b': u, 'h0': kvh * G, 'h1': (kvh + 1) * G, 'S': S, 'H': H, 'hd': hd},
                       [(part, (u * S * H, (u + 1) * S * H))], [(o, (u, u + 1), (kvh * G * hd, (kvh + 1) * G * hd))], prio, f'{p}merge.{u}.{kvh}')
        x1 = g.buffer(p + 'x1', B, d)
        gemv(p + 'o', o, 'wb.' + p + 'o', x1, d, H * hd, 0, res=x, prio=prio)
        gate, up = g.buffer(p + 'gate', B, F), g.buffer(p + 'up', B, F)
        r_gu = phase_rows([F, F], d)
        gemv(p + 'gate', x1, 'wb.' + p + 'gate', gate, F, d, 1, gamma='w.' + p + 'ln2', prio=prio, rows=r_gu)
        gemv(p + 'up', x1, 'wb.' + p + 'up', up, F, d, 1, gamma='w.' + p + 'ln2', prio=prio, rows=r_gu)
        xn = g.buffer(p + 'x2', B, d)
        gemv(p + 'down', gate, 'wb.' + p + 'down', xn, d, F, 2, x2=up, res=x1, prio=prio)
        x = xn
    logits = g.buffer('logits', B, V)
    gemv('head', x, 'wb.head', logits, V, d, 1, gamma='w.lnf', prio=1)
    g.task('argmax', {'logits': logits, 'out': tok, 'r0': 0, 'r1': B, 'V': V}, [logits], [tok], 1, 'argmax')
    g.task('counter_inc', {'x': lens, 'i0': 0, 'i1': B, 'delta': 1}, [lens], [lens], 0, 'advance')
    return g


def build_decode_tp(c: DecodeConfig, rank: int, world: int, exact: bool = False, fused: bool = False):
    """Rank `rank`'s share of the one-token graph under tensor parallelism over `world` ranks, batch 1.

    q / k / v / gate / up are sharded by output rows (heads, FFN columns), the o and down projections by input columns, the
    LM head by vocabulary rows; the KV cache holds the rank's kv heads.  The o and down projections therefore produce partial
    sums `[1, hidden]` that must be added over the ranks (the residual rides on rank 0's partial), which cuts the token into
    2 * layers + 1 segments.  Returns (graph, cuts, exchanges): cuts[i] = first task of segment i, exchanges[i] = name of the
    buffer to sum over the ranks after segment i (None after the last one, whose `logits` hold the rank's vocabulary slice).
    exact=True takes every shard as a slice of the full model's seeded weights (small configurations, parity tests);
    otherwise the shards are seeded on their own (same shapes and traffic, a different random model).

    fused=True keeps the token in ONE graph (one launch per token and rank): the sums over the ranks become tasks.  The o / down
    projection writes its partial to a buffer of its own; one peer_put_signal task per peer stores it into that peer's inbox row
    (site, this rank) and releases the flag word (site, this rank) with version lens + 1, and a peer_wait_sum task waits for the
    other ranks' flags and adds the partials in rank order (extension ops 302 / 303, include/kvm_ops.def).  The first buffers of
    the graph are `tp.inbox` [sites * world, hidden] and `tp.flag` [1, sites * world] (this rank's, written by the peers) and, per
    peer p, `tp.peer{p}.inbox` / `tp.peer{p}.flag`: the host binds those to the peers' memory before the first run.  cuts and
    exchanges then describe a single segment.
    """
    from .. import initgen
    P = world
    d, H, Hkv, hd, F, V, S = c.hidden, c.heads, c.kv_heads, c.head_dim, c.ffn, c.vocab, c.splits
    assert c.batch == 1 and H % P == 0 and Hkv % P == 0 and F % P == 0 and V % P == 0, 'heads, kv heads, ffn and vocab must divide by the ranks'
    Hl, Hkvl, Fl, Vl, G = H // P, Hkv // P, F // P, V // P, H // Hkv
    g = Graph('decode_tp')
    g.join_threshold = c.join_threshold
    seed_of = lambda name: zlib.crc32(f'{c.seed}/{name}'.encode())

    def full(name, n, k, scale):
        draws, bias, coef = initgen.seeded_params('normal', scale)
        return initgen.seeded_values(seed_of(name), n * k, draws, bias, coef).reshape(n, k)      # rounded to bf16 where it is stored

    def W(name, n, k, rows=None, cols=None):
        """bf16 weight shard: rows / cols = slice of the full [n, k] matrix held by this rank."""
        r0, r1 = rows or (0, n)
        c0, c1 = cols or (0, k)
        if exact:
            return g.data('wb.' + name, np.ascontiguousarray(full(name, n, k, c.init_std)[r0:r1, c0:c1]), 'bf16')
        return g.buffer('wb.' + name, r1 - r0, c1 - c0, 'bf16', {'kind': 'seeded', 'seed': seed_of(f'{name}/{rank}'), 'scale': c.init_std, 'dist': 'normal'})

    def gemv(tag, x, w, out, n, k, pro=0, x2=None, gamma=None, res=None, prio=20, rows=None):
        rows = rows or max(8, -(-n // c.workers)) if c.rows_per_task <= 0 else c.rows_per_task
        for i, n0 in enumerate(range(0, n, rows)):
            n1 = min(n0 + rows, n)
            g.task('gemv_bf16', {'x': x, 'x2': x2, 'gamma': gamma, 'w': w, 'out': out, 'res': res, 'n0': n0, 'n1': n1, 'K': k, 'pro': pro, 'eps': c.eps},
                   [x, x2, gamma, (w, (n0, n1)), (res, (0, 1), (n0, n1)) if res else None], [(out, (0, 1), (n0, n1))], prio, f'{tag}.{i}')

    sites = 2 * c.layers
    if fused:
        inbox, flag = g.buffer('tp.inbox', sites * P, d), g.buffer('tp.flag', 1, sites * P, 'i32')
        peers = {p: (g.buffer(f'tp.peer{p}.inbox', sites * P, d), g.buffer(f'tp.peer{p}.flag', 1, sites * P, 'i32')) for p in range(P) if p != rank}

    def exchange(site, partial, out, prio, tag):
        """out = sum over the ranks of their `partial`, inside the launch."""
        row0 = site * P
        for p, (pin, pfl) in peers.items():
            g.task('peer_put_signal', {'src': partial, 'dst': pin, 'src_off': 0, 'dst_off': (row0 + rank) * d, 'n': d, 'flag': pfl, 'var': row0 + rank, 'ver': 1,
                                       'seq': lens, 'stride': 1}, [partial, lens], [(pin, (row0 + rank, row0 + rank + 1)), (pfl, (0, 1), (row0 + rank, row0 + rank + 1))],
                   prio, f'{tag}.put{p}')
        g.task('peer_wait_sum', {'partial': partial, 'inbox': inbox, 'flag': flag, 'out': out, 'res': None, 'n': d, 'row0': row0, 'rank': rank, 'world': P, 'ver': 1,
                                 'seq': lens, 'stride': 1, 'p_off': 0, 'o_off': 0}, [partial, lens, (inbox, (row0, row0 + P)), (flag, (0, 1), (row0, row0 + P))], [out], prio, f'{tag}.sum')

    W('embed', V, d)
    g.buffer('w.lnf', 1, d, init={'kind': 'fill', 'value': 1.0})
    W('head', V, d, rows=(rank * Vl, (rank + 1) * Vl))
    lens = g.buffer('u0.lens', 1, 1, 'i32', {'kind': 'fill', 'value': c.ctx})
    tok = g.buffer('u0.tok', 1, 1, 'i32', {'kind': 'fill', 'value': 3 % V})
    x = g.buffer('u0.x', 1, d)
    cuts, exchanges = [0], []
    g.task('gather_rows', {'src': 'wb.embed', 'idx': tok, 'dst': x, 'r0': 0, 'r1': 1, 'd': d}, ['wb.embed', tok], [x], 31, 'u0.embed')
    for l in range(c.layers):
        p, tl = f'l{l}.', f'u0.l{l}.'
        prio = max(30 - l, 2)
        ln1 = g.buffer('w.' + p + 'ln1', 1, d, init={'kind': 'fill', 'value': 1.0})
        ln2 = g.buffer('w.' + p + 'ln2', 1, d, init={'kind': 'fill', 'value': 1.0})
        wq = W(p + 'q', H * hd, d, rows=(rank * Hl * hd, (rank + 1) * Hl * hd))
        wk = W(p + 'k', Hkv * hd, d, rows=(rank * Hkvl * hd, (rank + 1) * Hkvl * hd))
        wv = W(p + 'v', Hkv * hd, d, rows=(rank * Hkvl * hd, (rank + 1) * Hkvl * hd))
        wo = W(p + 'o', d, H * hd, cols=(rank * Hl * hd, (rank + 1) * Hl * hd))
        wg = W(p + 'gate', F, d, rows=(rank * Fl, (rank + 1) * Fl))
        wu = W(p + 'up', F, d, rows=(rank * Fl, (rank + 1) * Fl))
        wd = W(p + 'down', d, F, cols=(rank * Fl, (rank + 1) * Fl))
        # the cache of the rank's kv heads: a slice (by head) of the full model's seeded cache when exact
        if exact:
            cache = lambda n: g.data(tl + n, np.ascontiguousarray(full(f'u0.l{l}.{n}', Hkv * c.tmax, hd, 1.0)[rank * Hkvl * c.tmax:(rank + 1) * Hkvl * c.tmax]), 'bf16')
        else:
            cache = lambda n: g.buffer(tl + n, Hkvl * c.tmax, hd, 'bf16', {'kind': 'seeded', 'seed': seed_of(f'{tl}{n}/{rank}'), 'scale': 1.0, 'dist': 'normal'})
        kc, vc = cache('kc'), cache('vc')
        q, k, v = g.buffer(tl + 'q', 1, Hl * hd), g.buffer(tl + 'k', 1, Hkvl * hd), g.buffer(tl + 'v', 1, Hkvl * hd)
        rq = max(8, -(-(Hl + 2 * Hkvl) * hd // c.workers))
        gemv(tl + 'q', x, wq, q, Hl * hd, d, 1, gamma=ln1, prio=prio, rows=rq)
        gemv(tl + 'k', x, wk, k, Hkvl * hd, d, 1, gamma=ln1, prio=prio, rows=rq)
        gemv(tl + 'v', x, wv, v, Hkvl * hd, d, 1, gamma=ln1, prio=prio, rows=rq)
        part, o = g.buffer(tl + 'part', S * Hl, hd + 2), g.buffer(tl + 'o', 1, Hl * hd)
        slice_ = c.tmax // S
        for kvh in range(Hkvl):
            for s in range(S):
                rows = (kvh * c.tmax + s * slice_, kvh * c.tmax + (s + 1) * slice_)
                g.task('attn_decode_part', {'q': q, 'kc': kc, 'vc': vc, 'lens': lens, 'part': part, 'knew': k, 'vnew': v, 'b': 0, 'kvh': kvh, 's': s, 'S': S, 'H': Hl,
                                            'Hkv': Hkvl, 'hd': hd, 'Tmax': c.tmax, 'scale': hd ** -0.5, 'theta': c.theta, 'flags': 3},
                       [q, k, v, lens], [(kc, rows), (vc, rows), (part, (s * Hl + kvh * G, s * Hl + (kvh + 1) * G))], prio, f'{tl}part.{kvh}.{s}')
        for kvh in range(Hkvl):
            g.task('attn_decode_merge', {'part': part, 'o': o, 'b': 0, 'h0': kvh * G, 'h1': (kvh + 1) * G, 'S': S, 'H': Hl, 'hd': hd},
                   [part], [(o, (0, 1), (kvh * G * hd, (kvh + 1) * G * hd))], prio, f'{tl}merge.{kvh}')
        x1 = g.buffer(tl + 'x1', 1, d)               # partial sum of the o projection (+ residual on rank 0); summed over the ranks after the segment
        if fused:
            x1p = g.buffer(tl + 'x1p', 1, d)
            gemv(tl + 'o', o, wo, x1p, d, Hl * hd, 0, res=x if rank == 0 else None, prio=prio)
            exchange(2 * l, x1p, x1, prio, tl + 'x1')
        else:
            gemv(tl + 'o', o, wo, x1, d, Hl * hd, 0, res=x if rank == 0 else None, prio=prio)
            cuts.append(len(g.tasks)); exchanges.append(x1)
        gate, up = g.buffer(tl + 'gate', 1, Fl), g.buffer(tl + 'up', 1, Fl)
        rgu = max(8, -(-2 * Fl // c.workers))
        gemv(tl + 'gate', x1, wg, gate, Fl, d, 1, gamma=ln2, prio=prio, rows=rgu)
        gemv(tl + 'up', x1, wu, up, Fl, d, 1, gamma=ln2, prio=prio, rows=rgu)
        xn = g.buffer(tl + 'x2', 1, d)
        if fused:
            xnp = g.buffer(tl + 'x2p', 1, d)
            gemv(tl + 'down', gate, wd, xnp, d, Fl, 2, x2=up, res=x1 if rank == 0 else None, prio=prio)
            exchange(2 * l + 1, xnp, xn, prio, tl + 'x2')
        else:
            gemv(tl + 'down', gate, wd, xn, d, Fl, 2, x2=up, res=x1 if rank == 0 else None, prio=prio)
            cuts.append(len(g.tasks)); exchanges.append(xn)
        x = xn
    logits = g.buffer('u0.logits', 1, Vl)
    gemv('u0.head', x, 'wb.head', logits, Vl, d, 1, gamma='w.lnf', prio=1, rows=max(8, -(-Vl // (2 * c.workers))))
    g.task('counter_inc', {'x': lens, 'i0': 0, 'i1': 1, 'delta': 1}, [lens], [lens], 0, 'u0.advance')
    exchanges.append(None)
    return g, cuts, exchanges
