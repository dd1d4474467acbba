"""GPT training workloads in the reference's task ABI: a decoder-only pre-LN transformer (learned positions, GELU MLP,
optional tied head), forward + backward + global-norm clip + AdamW, emitted as tile tasks of the registered ops.

What the program computes per step follows the reference's training program (`frontend/mvmfe/train.py:145-190`: data
window -> forward -> loss -> backward -> clip -> step counter -> `pre` publish -> AdamW -> `post` publish, two publishes of
the `weights` variable per step) and its GPT block (`frontend/mvmfe/nn.py:187-210`), with the two variations the op set
provides for: learned absolute positions through `embedding_fwd`'s `wpe` (gradient: `embedding_bwd` with ids = -1, mod = T,
`include/mvm_ops_gpt.def:21-25`) and a tied head through `matmul_tile` flag 2 on `wte`.  Weights are `seeded normal`
buffers with seed crc32("<seed>/<param>") (`frontend/mvmfe/train.py:122-124`).

precision 'f32': f32 storage, `matmul_tile` (64x64 tiles).  precision 'bf16': f32 master weights and residual stream, bf16
storage for GEMM operands and activations, `matmul_mma_bf16` 128x256 tiles, weights re-rounded to bf16 shadows each step.
"""
from __future__ import annotations

import zlib
from dataclasses import dataclass, replace

import numpy as np

from .graph import Graph


@dataclass(frozen=True)
class GPTConfig:
    name: str = 'gpt_tiny'
    layers: int = 2
    d_model: int = 128
    heads: int = 4
    d_ff: int = 512
    vocab: int = 256
    seq: int = 64
    batch: int = 8
    tied: bool = True
    precision: str = 'f32'
    lr: float = 3e-4
    b1: float = 0.9
    b2: float = 0.999
    eps: float = 1e-8
    wd: float = 0.01
    clip: float = 1.0
    ln_eps: float = 1e-5
    init_std: float = 0.02
    seed: int = 0
    data_seed: int = 1
    # tiling
    norm_rows: int = 16
    ce_rows: int = 8
    flat_chunk: int = 65536
    col_chunk: int = 64
    key_chunk: int = 256
    join_threshold: int = 24  # a read with more producers than this waits on one join no-op instead of on each of them

    @property
    def tokens(self):
        return self.batch * self.seq


PRESETS = {
    # BASELINE config 1: runnable on the CPU oracle
    'gpt_tiny': GPTConfig(),
    'gpt_micro': GPTConfig(name='gpt_micro', layers=1, d_model=32, heads=2, d_ff=64, vocab=64, seq=16, batch=2, norm_rows=8, ce_rows=8,
                           flat_chunk=1024, col_chunk=16, key_chunk=32),
    # BASELINE config 3.  norm_rows 64: a norm / attention-delta phase of 8192 rows is 128 tasks, one wave over the SMs (16-row tasks
    # were mostly fixed cost: 512 tasks of 10 us per phase)
    'gpt_162m': GPTConfig(name='gpt_162m', layers=12, d_model=768, heads=12, d_ff=3072, vocab=50304, seq=1024, batch=8, tied=False,
                          precision='bf16', lr=6e-4, wd=0.1, flat_chunk=262144, norm_rows=64),
    # the 162M shapes at a size an ncu capture replays in seconds (2 layers, micro-batch 4): same tiles, same op mix
    'gpt_162m_2l': GPTConfig(name='gpt_162m_2l', layers=2, d_model=768, heads=12, d_ff=3072, vocab=50304, seq=1024, batch=4, tied=False,
                             precision='bf16', lr=6e-4, wd=0.1, flat_chunk=262144, norm_rows=32),
    # BASELINE config 4
    'gpt_355m': GPTConfig(name='gpt_355m', layers=24, d_model=1024, heads=16, d_ff=4096, vocab=50304, seq=1024, batch=8, tied=False,
                          precision='bf16', lr=6e-4, wd=0.1, flat_chunk=262144, norm_rows=64),
}


def preset(name: str, **over) -> GPTConfig:
    return replace(PRESETS[name], **over)


def token_stream(cfg: GPTConfig, steps: int, rank: int = 0, world: int = 1):
    """ids, tgt (int32 [steps*B*T]): uniform tokens in [0, V) from `data_seed`, next-token targets. Under data parallelism rank r
    of `world` takes microbatch r of each group of `world` (`runtime/partition.py:1349-1351` of the reference)."""
    rng = np.random.default_rng(cfg.data_seed)
    seqs = rng.integers(0, cfg.vocab, size=(steps * world, cfg.batch, cfg.seq + 1), dtype=np.int32)
    mine = seqs[rank::world]
    return mine[:, :, :-1].reshape(-1).copy(), mine[:, :, 1:].reshape(-1).copy()


def param_shapes(c: GPTConfig):
    """(name, rows, cols, fill or None, is a GEMM operand) of every parameter, in declaration order."""
    d = c.d_model
    out = [('wte', c.vocab, d, None, False), ('wpe', c.seq, d, None, False)]
    for l in range(c.layers):
        p = f'h{l}.'
        out += [(p + 'ln1.g', 1, d, 1.0, False), (p + 'ln1.b', 1, d, 0.0, False)]
        for n in 'qkv':
            out += [(p + f'attn.{n}.w', d, d, None, True), (p + f'attn.{n}.b', 1, d, 0.0, False)]
        out += [(p + 'attn.o.w', d, d, None, True), (p + 'attn.o.b', 1, d, 0.0, False)]
        out += [(p + 'ln2.g', 1, d, 1.0, False), (p + 'ln2.b', 1, d, 0.0, False)]
        out += [(p + 'fc.w', d, c.d_ff, None, True), (p + 'fc.b', 1, c.d_ff, 0.0, False)]
        out += [(p + 'proj.w', c.d_ff, d, None, True), (p + 'proj.b', 1, d, 0.0, False)]
    out += [('lnf.g', 1, d, 1.0, False), ('lnf.b', 1, d, 0.0, False)]
    if not c.tied:
        out.append(('head.w', d, c.vocab, None, True))
    return out


def dp_exchange_layout(c: GPTConfig, world: int):
    """Layout of the in-launch gradient exchange of data parallelism over `world` ranks, the same on every rank: the gradient arena
    ({parameter: element offset}, 64-element aligned, and its length), the exchange chunks [(parameter, e0, e1)] (the optimizer's
    own flat chunks: chunk k is summed by rank k % world), the inbox row length and the number of chunks a rank owns at most."""
    tmp = Graph('layout')
    off, arena, chunks = 0, {}, []
    for name, rows, cols, _, _ in param_shapes(c):
        tmp.buffer('w.' + name, rows, cols)
        arena[name] = off
        off += -(-rows * cols // 64) * 64
        chunks += [(name, e0, e1) for e0, e1 in tmp.flat_chunks('w.' + name, c.flat_chunk)]
    width = -(-max(e1 - e0 for _, e0, e1 in chunks) // 4) * 4
    return arena, off, chunks, width, -(-len(chunks) // world)


class _Emit:
    def __init__(self, cfg: GPTConfig, steps: int, rank=0, world=1, stream_steps=None, dp_fused=False):
        self.c, self.g = cfg, Graph('train')
        self.rank, self.world, self.dp_fused = rank, world, bool(dp_fused) and world > 1
        if self.dp_fused:
            # Buffers of the in-launch gradient exchange come first, so that a runner has this rank's exported ones before it binds
            # the peers' (kvm_b200/dp.py): the arena every gradient buffer is a slice of, the inbox the peers store their partial
            # chunks into (row = owned chunk * world + sending rank), its flag words, the flag words of the summed chunks coming back.
            _, n_arena, chunks, width, owned = dp_exchange_layout(cfg, world)
            gb = self.g.buffer
            gb('dp.arena', 1, n_arena), gb('dp.inbox', owned * world, width), gb('dp.flag', 1, owned * world, 'i32'), gb('dp.gflag', 1, len(chunks), 'i32')
            for p in range(world):
                if p != rank:
                    gb(f'dp.peer{p}.arena', 1, n_arena), gb(f'dp.peer{p}.inbox', owned * world, width)
                    gb(f'dp.peer{p}.flag', 1, owned * world, 'i32'), gb(f'dp.peer{p}.gflag', 1, len(chunks), 'i32')
        self.g.join_threshold = cfg.join_threshold
        self.bf = cfg.precision == 'bf16'
        self.act = 'bf16' if self.bf else 'f32'
        self.params: dict[str, tuple] = {}
        self.prio = 31
        c, g = cfg, self.g
        N, d = c.tokens, c.d_model
        ids, tgt = token_stream(c, stream_steps or steps, rank, world)
        g.stream('stream_ids', ids)
        g.stream('stream_tgt', tgt)
        g.buffer('opt_step', 1, 1, 'i32')
        g.buffer('clip_coef', 1, 2, init={'kind': 'fill', 'value': 1.0})
        g.buffer('version_token', 1, 1)      # one cell that chains the publishers of `weights` (post(s-1) -> pre(s) -> post(s))
        for name, rows, cols, fill, mat in param_shapes(c):
            self.param(name, rows, cols, fill, mat)
        if c.tied and self.bf:
            g.buffer('wb.wte', c.vocab, d, 'bf16')
        for s in range(steps):
            self.step(s)

    # ---- parameters
    def param(self, name, rows, cols, fill=None, mat=False):
        g, c = self.g, self.c
        init = {'kind': 'fill', 'value': fill} if fill is not None else \
            {'kind': 'seeded', 'seed': zlib.crc32(f'{c.seed}/{name}'.encode()), 'scale': c.init_std, 'dist': 'normal'}
        g.buffer('w.' + name, rows, cols, init=init)
        g.buffer('m.' + name, rows, cols)
        g.buffer('v.' + name, rows, cols)
        g.buffer('g.' + name, rows, cols)
        if mat and self.bf:
            g.buffer('wb.' + name, rows, cols, 'bf16')
        self.params[name] = (rows, cols, mat)

    def W(self, name):
        """The GEMM operand holding parameter `name`."""
        return ('wb.' if self.bf else 'w.') + name

    # ---- op helpers (each emits the tile tasks of one logical op)
    def flat(self, op, bufs_r, bufs_w, n_elems, args, tag):
        """Elementwise op over equally shaped buffers, chunked on row boundaries."""
        g = self.g
        for i, (e0, e1) in enumerate(g.flat_chunks(bufs_w[0], self.c.flat_chunk)):
            rd = [(b, *g.region_of(b, e0, e1)) for b in bufs_r]
            wr = [(b, *g.region_of(b, e0, e1)) for b in bufs_w]
            g.task(op, {**args, 'e0': e0, 'e1': e1}, rd, wr, self.prio, f'{tag}.{i}')

    def linear(self, tag, a, w, out, M, N, K, flags=0, bias=None, res=None, pre=None, alpha=1.0):
        """out[M,N] (+)= alpha * op(a) op(w) (+bias) (gelu) (+res), tiled. Region reads follow the transposes."""
        g = self.g
        if self.bf:
            op, tm, tn = 'matmul_mma_bf16', 128, 256
        else:
            op, tm, tn = 'matmul_tile', 64, 64
        ta, tb, acc = flags & 1, flags & 2, flags & 4
        for m0 in range(0, M, tm):
            m1 = min(m0 + tm, M)
            for n0 in range(0, N, tn):
                n1 = min(n0 + tn, N)
                rd = [(a, (0, K), (m0, m1)) if ta else (a, (m0, m1), (0, K)),
                      (w, (n0, n1), (0, K)) if tb else (w, (0, K), (n0, n1))]
                if bias:
                    rd.append((bias, (0, 1), (n0, n1)))
                if res:
                    rd.append((res, (m0, m1), (n0, n1)))
                if acc:
                    rd.append((out, (m0, m1), (n0, n1)))
                wr = [(out, (m0, m1), (n0, n1))]
                if pre:
                    wr.append((pre, (m0, m1), (n0, n1)))
                g.task(op, {'a': a, 'b': w, 'out': out, 'bias': bias, 'res': res, 'pre': pre, 'm0': m0, 'n0': n0, 'M': M, 'N': N, 'K': K,
                            'flags': flags, 'alpha': alpha}, rd, wr, min(self.prio, 7) if ta else self.prio, f'{tag}.{m0 // tm}.{n0 // tn}')

    def rows(self, op, tag, N, per, args, reads, writes, vec_r=(), vec_w=()):
        """Row-block tasks over [0,N): matrices in reads/writes are touched on rows [r0,r1); vec_* are [N]-long flat vectors."""
        g = self.g
        for r0 in range(0, N, per):
            r1 = min(r0 + per, N)
            rd = [(b, (r0, r1)) if b in self._rowwise else b for b in reads if b] + [(b, g.rows_of(b, r0, r1)) for b in vec_r]
            wr = [(b, (r0, r1)) for b in writes] + [(b, g.rows_of(b, r0, r1)) for b in vec_w]
            g.task(op, {**args, 'r0': r0, 'r1': r1}, rd, wr, self.prio, f'{tag}.{r0 // per}')

    def layernorm(self, tag, x, gname, bname, out, mean, rstd):
        c = self.c
        self._rowwise = {x}
        self.rows('layernorm_fwd', tag, c.tokens, c.norm_rows,
                  {'x': x, 'gamma': gname, 'beta': bname, 'out': out, 'mean': mean, 'rstd': rstd, 'd': c.d_model, 'eps': c.ln_eps},
                  [x, gname, bname], [out], vec_w=[mean, rstd])

    def layernorm_bwd(self, tag, x, dy, pname, mean, rstd, dx, acc):
        c, g = self.c, self.g
        d, N = c.d_model, c.tokens
        self._rowwise = {x, dy, dx}
        self.rows('layernorm_bwd_dx', tag + '.dx', N, c.norm_rows,
                  {'x': x, 'dy': dy, 'gamma': 'w.' + pname + '.g', 'mean': mean, 'rstd': rstd, 'dx': dx, 'd': d, 'acc': acc},
                  [x, dy, 'w.' + pname + '.g'] + ([dx] if acc else []), [dx], vec_r=[mean, rstd])
        for c0 in range(0, d, c.col_chunk):
            c1 = min(c0 + c.col_chunk, d)
            g.task('norm_bwd_params', {'x': x, 'dy': dy, 'mean': mean, 'rstd': rstd, 'dgamma': 'g.' + pname + '.g', 'dbeta': 'g.' + pname + '.b',
                                       'R': N, 'd': d, 'c0': c0, 'c1': c1, 'acc': 0},
                   [(x, (0, N), (c0, c1)), (dy, (0, N), (c0, c1)), mean, rstd],
                   [('g.' + pname + '.g', (0, 1), (c0, c1)), ('g.' + pname + '.b', (0, 1), (c0, c1))], max(self.prio - 8, 0), f'{tag}.params.{c0}')

    def colsum(self, tag, x, out, R, ncols):
        g, ch = self.g, self.c.col_chunk
        for c0 in range(0, ncols, ch):
            c1 = min(c0 + ch, ncols)
            g.task('colsum', {'x': x, 'out': out, 'R': R, 'c0': c0, 'c1': c1, 'acc': 0}, [(x, (0, R), (c0, c1))], [(out, (0, 1), (c0, c1))],
                   max(self.prio - 8, 0), f'{tag}.{c0}')

    def to_operand(self, tag, x, rows, cols):
        """bf16 copy of an f32 tensor that a GEMM reads (bf16 precision only)."""
        if not self.bf:
            return x
        xb = self.g.buffer(x + '.bf', rows, cols, 'bf16')
        self.flat('round_bf16', [x], [xb], rows * cols, {'x': x, 'out': xb}, tag)
        return xb

    def attention(self, tag, q, k, v, o, lse):
        c, g = self.c, self.g
        T, H, hd = c.seq, c.heads, c.d_model // c.heads
        for b in range(c.batch):
            for h in range(H):
                cs = (h * hd, (h + 1) * hd)
                for q0 in range(0, T, 128):
                    q1 = min(q0 + 128, T)
                    g.task('attn_fwd', {'q': q, 'k': k, 'v': v, 'o': o, 'lse': lse, 'b': b, 'h': h, 'q0': q0, 'T': T, 'H': H, 'Hkv': H, 'hd': hd,
                                        'scale': hd ** -0.5},
                           [(q, (b * T + q0, b * T + q1), cs), (k, (b * T, b * T + q1), cs), (v, (b * T, b * T + q1), cs)],
                           [(o, (b * T + q0, b * T + q1), cs), (lse, g.rows_of(lse, (b * H + h) * T + q0, (b * H + h) * T + q1))],
                           self.prio, f'{tag}.{b}.{h}.{q0 // 128}')

    def attention_bwd(self, tag, q, k, v, o, lse, do, delta, dq, dk, dv):
        c, g = self.c, self.g
        T, H, hd, N = c.seq, c.heads, c.d_model // c.heads, c.tokens
        per = max(c.norm_rows, 1)
        for r0 in range(0, N, per):
            r1 = min(r0 + per, N)
            b0, b1 = r0 // T, (r1 - 1) // T + 1
            if b1 == b0 + 1:      # one sequence: the H strided pieces this block writes, (b*H+h)*T + t
                wr = [(delta, ((b0 * H + h) * T + r0 % T, (b0 * H + h) * T + r0 % T + (r1 - r0))) for h in range(H)]
            else:
                wr = [(delta, (b0 * H * T, b1 * H * T))]
            g.task('attn_bwd_delta', {'o': o, 'do': do, 'delta': delta, 'r0': r0, 'r1': r1, 'T': T, 'H': H, 'hd': hd},
                   [(o, (r0, r1)), (do, (r0, r1))], wr, self.prio, f'{tag}.delta.{r0 // per}')
        sc = hd ** -0.5
        for b in range(c.batch):
            for h in range(H):
                cs = (h * hd, (h + 1) * hd)
                vec = g.rows_of(lse, (b * H + h) * T, (b * H + h + 1) * T)
                for q0 in range(0, T, 128):
                    q1 = min(q0 + 128, T)
                    g.task('attn_bwd_dq', {'q': q, 'k': k, 'v': v, 'do': do, 'lse': lse, 'delta': delta, 'dq': dq, 'b': b, 'h': h, 'q0': q0, 'T': T,
                                           'H': H, 'Hkv': H, 'hd': hd, 'scale': sc},
                           [(q, (b * T + q0, b * T + q1), cs), (k, (b * T, b * T + q1), cs), (v, (b * T, b * T + q1), cs),
                            (do, (b * T + q0, b * T + q1), cs), (lse, vec), (delta, vec)],
                           [(dq, (b * T + q0, b * T + q1), cs)], self.prio, f'{tag}.dq.{b}.{h}.{q0 // 128}')
                for k0 in range(0, T, 128):
                    k1 = min(k0 + 128, T)
                    g.task('attn_bwd_dkv', {'q': q, 'k': k, 'v': v, 'do': do, 'lse': lse, 'delta': delta, 'dk': dk, 'dv': dv, 'b': b, 'kvh': h,
                                            'k0': k0, 'T': T, 'H': H, 'hd': hd, 'scale': sc},
                           [(q, (b * T + k0, b * T + T), cs), (do, (b * T + k0, b * T + T), cs), (k, (b * T + k0, b * T + k1), cs),
                            (v, (b * T + k0, b * T + k1), cs), (lse, vec), (delta, vec)],
                           [(dk, (b * T + k0, b * T + k1), cs), (dv, (b * T + k0, b * T + k1), cs)], self.prio, f'{tag}.dkv.{b}.{h}.{k0 // 128}')

    # ---- one optimizer step
    def step(self, s):
        c, g, act = self.c, self.g, self.act
        N, d, F, V, T, L = c.tokens, c.d_model, c.d_ff, c.vocab, c.seq, c.layers
        B = g.buffer
        tag = f's{s}/'
        self.prio = 31
        if self.bf:
            for name, (rows, cols, mat) in self.params.items():
                if mat:
                    self.flat('round_bf16', ['w.' + name], ['wb.' + name], rows * cols, {'x': 'w.' + name, 'out': 'wb.' + name}, tag + 'shadow.' + name)
            if c.tied:
                self.flat('round_bf16', ['w.wte'], ['wb.wte'], V * d, {'x': 'w.wte', 'out': 'wb.wte'}, tag + 'shadow.wte')
        ids, tgt = B('ids', N, 1, 'i32'), B('tgt', N, 1, 'i32')
        for src, dst in (('stream_ids', ids), ('stream_tgt', tgt)):
            g.task('select_window', {'src': src, 'step': 'opt_step', 'dst': dst, 'i0': 0, 'i1': N, 'stride': N, 'off': 0},
                   ['opt_step'], [dst], self.prio, f'{tag}window.{dst}')
        x = B('x0', N, d)
        self._rowwise = {x}
        self.rows('embedding_fwd', tag + 'embed', N, 4 * c.norm_rows, {'ids': ids, 'wte': 'w.wte', 'wpe': 'w.wpe', 'out': x, 'T': T, 'd': d},
                  ['w.wte', 'w.wpe'], [x], vec_r=[ids])
        saved = []
        for l in range(L):
            p, t = f'h{l}.', f'{tag}h{l}.'
            self.prio = max(30 - l, 16)
            h1, mu1, rs1 = B(p + 'h1', N, d, act), B(p + 'mu1', N, 1), B(p + 'rs1', N, 1)
            self.layernorm(t + 'ln1', x, 'w.' + p + 'ln1.g', 'w.' + p + 'ln1.b', h1, mu1, rs1)
            q, k, v = (B(p + n, N, d, act) for n in 'qkv')
            for n, o_ in zip('qkv', (q, k, v)):
                self.linear(t + n, h1, self.W(p + f'attn.{n}.w'), o_, N, d, d, bias='w.' + p + f'attn.{n}.b')
            o, lse = B(p + 'o', N, d, act), B(p + 'lse', c.batch * c.heads * T, 1)
            self.attention(t + 'attn', q, k, v, o, lse)
            xm = B(p + 'xm', N, d)
            self.linear(t + 'o', o, self.W(p + 'attn.o.w'), xm, N, d, d, bias='w.' + p + 'attn.o.b', res=x)
            h2, mu2, rs2 = B(p + 'h2', N, d, act), B(p + 'mu2', N, 1), B(p + 'rs2', N, 1)
            self.layernorm(t + 'ln2', xm, 'w.' + p + 'ln2.g', 'w.' + p + 'ln2.b', h2, mu2, rs2)
            pre, a = B(p + 'pre', N, F, act), B(p + 'a', N, F, act)
            self.linear(t + 'fc', h2, self.W(p + 'fc.w'), a, N, F, d, flags=8, bias='w.' + p + 'fc.b', pre=pre)
            xo = B(p + 'xo', N, d)
            self.linear(t + 'proj', a, self.W(p + 'proj.w'), xo, N, d, F, bias='w.' + p + 'proj.b', res=xm)
            saved.append((x, h1, mu1, rs1, q, k, v, o, lse, xm, h2, mu2, rs2, pre, a))
            x = xo
        self.prio = 23
        hf, muf, rsf = B('hf', N, d, act), B('muf', N, 1), B('rsf', N, 1)
        self.layernorm(tag + 'lnf', x, 'w.lnf.g', 'w.lnf.b', hf, muf, rsf)
        logits = B('logits', N, V, act)
        if c.tied:
            self.linear(tag + 'head', hf, self.W('wte'), logits, N, V, d, flags=2)
        else:
            self.linear(tag + 'head', hf, self.W('head.w'), logits, N, V, d)
        rowloss, lse_ce, dlog = B('rowloss', N, 1), B('lse_ce', N, 1), B('dlogits', N, V, act)
        self._rowwise = {logits}
        self.rows('softmax_ce_fused', tag + 'ce', N, c.ce_rows,
                  {'logits': logits, 'tgt': tgt, 'rowloss': rowloss, 'lse': lse_ce, 'dlogits': dlog, 'V': V, 'ignore': -1, 'N': N,
                   'scale': 1.0 / self.world if self.dp_fused else 1.0},      # fused data parallelism: the mean over the ranks is folded into the loss gradient
                  [logits], [dlog], vec_r=[tgt], vec_w=[rowloss, lse_ce])
        loss = B(f'loss.{s}', 1, 2)
        g.task('softmax_ce_reduce', {'rowloss': rowloss, 'tgt': tgt, 'loss': loss, 'N': N, 'ignore': -1}, [rowloss, tgt], [loss], 0, tag + 'loss')

        # ---------------- backward
        # backward: the chain of input-gradient ops is the critical path (class 1); weight / bias / norm-parameter gradients only feed
        # the optimizer and run as filler (class 0: the ready queue serves higher classes first)
        self.prio = 15
        dhf = B('dhf', N, d, act)
        if c.tied:
            self.linear(tag + 'head.dx', dlog, self.W('wte'), dhf, N, d, V)
            self.linear(tag + 'head.dw', dlog, hf, 'g.wte', V, d, N, flags=1)
        else:
            self.linear(tag + 'head.dx', dlog, self.W('head.w'), dhf, N, d, V, flags=2)
            self.linear(tag + 'head.dw', hf, dlog, 'g.head.w', d, V, N, flags=1)
        dres = B('dres', N, d)
        self.layernorm_bwd(tag + 'lnf.bwd', x, dhf, 'lnf', muf, rsf, dres, 0)
        for l in reversed(range(L)):
            p, t = f'h{l}.', f'{tag}h{l}.bwd.'
            self.prio = 15
            x_in, h1, mu1, rs1, q, k, v, o, lse, xm, h2, mu2, rs2, pre, a = saved[l]
            dres_op = self.to_operand(t + 'dres.bf', dres, N, d)
            da = B('da', N, F, act)
            self.linear(t + 'proj.dx', dres_op, self.W(p + 'proj.w'), da, N, F, d, flags=2)
            self.linear(t + 'proj.dw', a, dres_op, 'g.' + p + 'proj.w', F, d, N, flags=1)
            self.colsum(t + 'proj.db', dres, 'g.' + p + 'proj.b', N, d)
            dpre = B('dpre', N, F, act)
            self.flat('gelu_bwd', [pre, da], [dpre], N * F, {'x': pre, 'dy': da, 'dx': dpre, 'acc': 0}, t + 'gelu')
            dh2 = B('dh2', N, d, act)
            self.linear(t + 'fc.dx', dpre, self.W(p + 'fc.w'), dh2, N, d, F, flags=2)
            self.linear(t + 'fc.dw', h2, dpre, 'g.' + p + 'fc.w', d, F, N, flags=1)
            self.colsum(t + 'fc.db', dpre, 'g.' + p + 'fc.b', N, F)
            self.layernorm_bwd(t + 'ln2', xm, dh2, p + 'ln2', mu2, rs2, dres, 1)
            dres_op = self.to_operand(t + 'dres2.bf', dres, N, d)
            do = B('do', N, d, act)
            self.linear(t + 'o.dx', dres_op, self.W(p + 'attn.o.w'), do, N, d, d, flags=2)
            self.linear(t + 'o.dw', o, dres_op, 'g.' + p + 'attn.o.w', d, d, N, flags=1)
            self.colsum(t + 'o.db', dres, 'g.' + p + 'attn.o.b', N, d)
            delta = B('delta', c.batch * c.heads * T, 1)
            dq, dk, dv = (B('d' + n, N, d, act) for n in 'qkv')
            self.attention_bwd(t + 'attn', q, k, v, o, lse, do, delta, dq, dk, dv)
            dh1 = B('dh1', N, d, act)
            for i, (n, dn) in enumerate(zip('qkv', (dq, dk, dv))):
                self.linear(t + n + '.dx', dn, self.W(p + f'attn.{n}.w'), dh1, N, d, d, flags=2 | (4 if i else 0))
                self.linear(t + n + '.dw', h1, dn, 'g.' + p + f'attn.{n}.w', d, d, N, flags=1)
                self.colsum(t + n + '.db', dn, 'g.' + p + f'attn.{n}.b', N, d)
            self.layernorm_bwd(t + 'ln1', x_in, dh1, p + 'ln1', mu1, rs1, dres, 1)
        self.prio = 2
        for v0 in range(0, V, c.key_chunk):
            v1 = min(v0 + c.key_chunk, V)
            g.task('embedding_bwd', {'ids': ids, 'dout': dres, 'dtab': 'g.wte', 'N': N, 'mod': 0, 'v0': v0, 'v1': v1, 'd': d, 'acc': 1 if c.tied else 0},
                   [ids, dres, ('g.wte', (v0, v1))] if c.tied else [ids, dres], [('g.wte', (v0, v1))], self.prio, f'{tag}embed.bwd.{v0}')
        pos_chunk = max(1, min(c.key_chunk, T // 32 if T >= 64 else T))
        for v0 in range(0, T, pos_chunk):
            v1 = min(v0 + pos_chunk, T)
            g.task('embedding_bwd', {'ids': None, 'dout': dres, 'dtab': 'g.wpe', 'N': N, 'mod': T, 'v0': v0, 'v1': v1, 'd': d, 'acc': 0},
                   [dres], [('g.wpe', (v0, v1))], self.prio, f'{tag}pos.bwd.{v0}')

        g.split_at = len(g.tasks)       # data parallelism: the gradient all-reduce sits here, between backward and the optimizer
        # ---------------- clip + AdamW, bracketed by the two publishes of `weights`
        chunks = []
        for name, (rows, cols, _) in self.params.items():
            for e0, e1 in g.flat_chunks('w.' + name, c.flat_chunk):
                chunks.append((name, e0, e1))
        if self.dp_fused:
            self.dp_exchange(tag, chunks)
        partial = B('gn_partial', 1, len(chunks))
        for slot, (name, e0, e1) in enumerate(chunks):
            g.task('gradnorm_partial', {'g': 'g.' + name, 'partial': partial, 'slot': slot, 'e0': e0, 'e1': e1},
                   [('g.' + name, *g.region_of('g.' + name, e0, e1))], [(partial, (0, 1), (slot, slot + 1))], 2, f'{tag}gnorm.{slot}')
        g.task('gradnorm_finish', {'partial': partial, 'nslots': len(chunks), 'out': 'clip_coef', 'max_norm': c.clip}, [partial], ['clip_coef'],
               2, tag + 'gnorm.finish')
        g.task('counter_inc', {'x': 'opt_step', 'i0': 0, 'i1': 1, 'delta': 1}, ['opt_step'], ['opt_step'], 2, tag + 'step_inc')
        grads = ['g.' + n for n in self.params]
        pre_id = g.task('noop', {}, grads + ['clip_coef', 'opt_step'], ['version_token'], 2, tag + 'barrier.pre', publishes='weights')
        ups = []
        for name, e0, e1 in chunks:
            wd = c.wd if self.params[name][2] or name in ('wte', 'wpe') else 0.0
            rr = g.region_of('w.' + name, e0, e1)
            ups.append(g.task('adamw', {'p': 'w.' + name, 'g': 'g.' + name, 'm': 'm.' + name, 'v': 'v.' + name, 'gscale': 'clip_coef', 'step': 'opt_step',
                                        'e0': e0, 'e1': e1, 'lr': c.lr, 'b1': c.b1, 'b2': c.b2, 'eps': c.eps, 'wd': wd},
                              [('g.' + name, *rr), 'clip_coef', 'opt_step'], [('w.' + name, *rr), ('m.' + name, *rr), ('v.' + name, *rr)], 1,
                              f'{tag}adamw.{name}.{e0}', after=[pre_id]))
        g.task('noop', {}, [], ['version_token'], 1, tag + 'barrier.post', publishes='weights', after=ups)


    def dp_exchange(self, tag, chunks):
        """The gradient all-reduce (mean) of data parallelism as tasks of the step, between the backward and the optimizer: chunk k of
        the gradients is owned by rank k % world.  Every other rank stores its chunk into the owner's inbox and releases a flag
        (peer_put_signal); the owner waits for the world - 1 flags, adds the partials in rank order in place (peer_wait_sum) and
        stores the sum into every peer's gradient arena, releasing that peer's flag of the chunk; a non-owner waits for that flag
        (peer_wait) before anything reads the chunk.  Versions are the optimizer step counter + 1.  The 1 / world of the mean is in
        the loss gradient already.  The tasks are ordinary low-priority tasks: they run while the backward still has work."""
        g, P, rank = self.g, self.world, self.rank
        arena, _, layout_chunks, width, owned = dp_exchange_layout(self.c, P)
        assert layout_chunks == chunks
        seq = {'seq': 'opt_step', 'stride': 1, 'ver': 1}
        sends, recvs = [], []
        for k, (name, e0, e1) in enumerate(chunks):
            gbuf, n = 'g.' + name, e1 - e0
            region = (gbuf, *g.region_of(gbuf, e0, e1))
            owner, j = k % P, k // P
            if owner == rank:
                g.task('peer_wait_sum', {'partial': gbuf, 'inbox': 'dp.inbox', 'flag': 'dp.flag', 'out': gbuf, 'res': None, 'n': n, 'row0': j * P, 'rank': rank,
                                         'world': P, **seq, 'p_off': e0, 'o_off': e0}, [region, 'opt_step'], [region], 2, f'{tag}dp.sum.{k}')
                for p in range(P):
                    if p != rank:
                        g.task('peer_put_signal', {'src': gbuf, 'dst': f'dp.peer{p}.arena', 'src_off': e0, 'dst_off': arena[name] + e0, 'n': n,
                                                   'flag': f'dp.peer{p}.gflag', 'var': k, **seq}, [region, 'opt_step'], [], 2, f'{tag}dp.bcast.{k}.{p}')
            else:
                sends.append(g.task('peer_put_signal', {'src': gbuf, 'dst': f'dp.peer{owner}.inbox', 'src_off': e0, 'dst_off': (j * P + rank) * width, 'n': n,
                                                        'flag': f'dp.peer{owner}.flag', 'var': j * P + rank, **seq}, [region, 'opt_step'], [], 2, f'{tag}dp.send.{k}'))
                recvs.append((k, region))
        # A wait occupies its worker until the flag comes.  The waits for the sums coming back are therefore held until this rank has
        # sent its last chunk (the backward is over then, and most sums have arrived long before): they cost a poll each, not a stall.
        sent = g.task('noop', {}, [], [], 2, f'{tag}dp.sent', after=sends) if sends else None
        for k, region in recvs:
            g.task('peer_wait', {'flag': 'dp.gflag', 'row0': k, 'count': 1, **seq}, [region, 'opt_step'], [region], 2, f'{tag}dp.recv.{k}', after=[sent])


def build_training(cfg: GPTConfig, steps: int = 1, rank: int = 0, world: int = 1, stream_steps: int | None = None, dp_fused: bool = False) -> Graph:
    """`steps` optimizer steps unrolled in one graph; the token stream holds `stream_steps` (default `steps`) windows, so a
    one-step graph can be re-run `stream_steps` times (the device step counter selects the window).  dp_fused: with world > 1 the
    gradient all-reduce is part of the graph (`_Emit.dp_exchange`), one launch per step and rank."""
    return _Emit(cfg, steps, rank, world, stream_steps, dp_fused).g
