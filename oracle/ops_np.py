"""CPU oracle: numpy restatement of the reference's per-op semantics.  TEST INFRASTRUCTURE, not product code.

Only tests/, `__graft_entry__.smoke()` and `bench.py`'s cpu_baseline / `--impl reference` legs may import this package;
the executor (kvm_b200/) never does and has no CPU fallback.

Every function restates one reference operator with the SAME rounding points, vectorised instead of scalar loops:
  core ops              runtime/ref_ops.py:17-84
  GPT pack              runtime/ref_gpt.py:44-613
  bf16 / decode / misc  runtime/ref_extra.py:56-80,312-415,421-498
Rule of the reference model (runtime/ref_gpt.py:1-7): operands and results are float32 values; reductions and
transcendentals run in double; every stored result is rounded to float32 once; AdamW / SGD / colsum / embedding_bwd /
matmul follow a strict float32 step order.  A value stored into a bf16 buffer (ABI dtype 2) is additionally rounded to
bfloat16, nearest-even, once (include/mvm_ops_extra.def:63-70).

Pinned against the reference in tests/test_oracle_golden.py: known-answer vectors of the reference's own tests
(SplitMix64, Philox) and fixtures produced by importing the reference's pure-Python ops (tests/golden/make_golden.py).

Buffers are `Buf` objects: a 2-D numpy array (float32 for f32 and bf16 storage, int32 for i32) plus the ABI dtype code.
`exact_matmul=True` reproduces the reference's k-ascending float32 accumulation bit for bit; False uses BLAS sgemm on
the (already rounded) operands, which is what the timed CPU baseline uses at model sizes.
"""
from __future__ import annotations

import math

import numpy as np

F32, I32, BF16 = 0, 1, 2
ATTN_ROWS = 128                      # runtime/ref_gpt.py:14
ATTN_EMPTY_M = np.float32(-3.4028234663852886e38)   # runtime/ref_extra.py:417
f32 = np.float32
f64 = np.float64


class OracleError(ValueError):
    """An argument no execution could accept (the reference raises ValueError; the device reports an op error)."""


class Buf:
    __slots__ = ('a', 'dtype')

    def __init__(self, a: np.ndarray, dtype: int):
        self.a, self.dtype = a, dtype

    @property
    def rows(self):
        return self.a.shape[0]

    @property
    def cols(self):
        return self.a.shape[1]

    @property
    def flat(self):
        return self.a.reshape(-1)


def bf16_round(x):
    """float32 -> nearest bfloat16 value, ties to even, inf/nan kept (runtime/ref_extra.py:41-47)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    bits = x.view(np.uint32)
    r = ((bits + np.uint32(0x7FFF) + ((bits >> np.uint32(16)) & np.uint32(1))) & np.uint32(0xFFFF0000)).view(np.float32)
    return np.where(np.isfinite(x), r, x)


def tf32_round(x):
    """To nearest, ties away, low 13 bits cleared; NaN keeps its high bits (runtime/ref_gpt.py:217-223)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    u = x.view(np.uint32)
    u = np.where((u & np.uint32(0x7FFFFFFF)) <= np.uint32(0x7F800000), u + np.uint32(0x1000), u)
    return (u & np.uint32(0xFFFFE000)).view(np.float32)


def _st(buf: Buf, v):
    """Value(s) as stored into `buf`: float32, then bf16 for bf16 storage."""
    v = np.asarray(v).astype(np.float32)
    return bf16_round(v) if buf.dtype == BF16 else v


def _need(c, msg):
    if not c:
        raise OracleError(msg)


def _gelu(x):
    x = x.astype(f64)
    return 0.5 * x * (1.0 + np.tanh(0.7978845608028654 * (x + 0.044715 * x * x * x)))


def _gelu_grad(x):
    x = x.astype(f64)
    t = np.tanh(0.7978845608028654 * (x + 0.044715 * x * x * x))
    return 0.5 * (1 + t) + 0.5 * x * (1 - t * t) * 0.7978845608028654 * (1 + 3 * 0.044715 * x * x)


def _sig(x):
    x = x.astype(f64)
    e = np.exp(-np.abs(x))
    return np.where(x >= 0, 1.0 / (1.0 + e), e / (1.0 + e))


def _silu(x):
    return x.astype(f64) * _sig(x)


def _silu_d(x):
    s = _sig(x)
    return s * (1.0 + x.astype(f64) * (1.0 - s))


# ---- core ----------------------------------------------------------------------------------------------------------------
def noop(b, a, **kw):
    pass


def copy(b, a, **kw):
    b['dst'].flat[:a['n']] = b['src'].flat[:a['n']]


def add(b, a, **kw):
    n = a['n']
    b['out'].flat[:n] = _st(b['out'], b['a'].flat[:n] + b['b'].flat[:n])


def scale(b, a, **kw):
    n = a['n']
    b['out'].flat[:n] = _st(b['out'], b['x'].flat[:n] * f32(a['alpha']))


def relu(b, a, **kw):
    n = a['n']
    x = b['x'].flat[:n]
    b['out'].flat[:n] = np.where(x > 0, x, f32(0))


def sgd(b, a, **kw):
    n = a['n']
    w = b['w'].flat
    w[:n] = w[:n] - f32(a['lr']) * b['g'].flat[:n]


def predict(b, a, **kw):
    n = a['n']
    b['out'].flat[:n] = b['w'].flat[0] * b['x'].flat[:n]


def mse_grad(b, a, **kw):
    n = a['n']
    d = b['pred'].flat[:n] - b['target'].flat[:n]
    la = ga = f32(0)
    t1, t2 = d * d, (f32(2.0) * d) * b['x'].flat[:n]
    for i in range(n):
        la, ga = f32(la + t1[i]), f32(ga + t2[i])
    b['loss'].flat[0] = f32(f64(la) / n)
    b['grad'].flat[0] = f32(f64(ga) / n)


def _mm_seq(A, B):
    """acc = f32(acc + f32(x*y)), k ascending: the reference's exact-product golden (runtime/ref_gpt.py:78-82)."""
    acc = np.zeros((A.shape[0], B.shape[1]), np.float32)
    for k in range(A.shape[1]):
        acc += A[:, k:k + 1] * B[k:k + 1, :]
    return acc


def matmul(b, a, **kw):
    m, n, k = a['m'], a['n'], a['k']
    A, B = b['a'].flat[:m * k].reshape(m, k), b['b'].flat[:k * n].reshape(k, n)
    b['out'].flat[:m * n] = (_mm_seq(A, B) if kw.get('exact_matmul', True) else A @ B).reshape(-1)


def fill(b, a, **kw):
    b['x'].flat[:a['n']] = a['value']


def spin(b, a, **kw):
    pass


# ---- embeddings ----------------------------------------------------------------------------------------------------------
def embedding_fwd(b, a, **kw):
    ids, wte, wpe, out = b['ids'], b['wte'], b['wpe'], b['out']
    r0, r1, d, T = a['r0'], a['r1'], a['d'], a['T']
    tok = ids.flat[r0:r1]
    _need(((tok >= 0) & (tok < wte.rows)).all(), 'embedding_fwd: token id outside [0,V)')
    v = wte.a[tok, :d]
    if wpe is not None:
        v = v + wpe.a[np.arange(r0, r1) % T, :d]
    out.a[r0:r1, :d] = _st(out, v)


def embedding_bwd(b, a, **kw):
    ids, dout, dt = b['ids'], b['dout'], b['dtab']
    N, mod, v0, v1, d = a['N'], a['mod'], a['v0'], a['v1'], a['d']
    _need(ids is not None or mod > 0, 'embedding_bwd: ids absent needs mod > 0')
    keys = ids.flat[:N] if ids is not None else np.arange(N) % mod
    acc = dt.a[v0:v1, :d].astype(np.float32) if a['acc'] else np.zeros((v1 - v0, d), np.float32)
    g = dout.a[:N, :d]
    sel = np.flatnonzero((keys >= v0) & (keys < v1))
    # rows ascending per key, one float32 add each (runtime/ref_gpt.py:58-65): stable sort by key keeps row order
    order = sel[np.argsort(keys[sel], kind='stable')]
    ks = keys[order] - v0
    if len(order):
        starts = np.flatnonzero(np.r_[True, ks[1:] != ks[:-1]])
        lens = np.diff(np.r_[starts, len(ks)])
        for j in range(int(lens.max())):
            live = starts[lens > j] + j
            acc[ks[live]] += g[order[live]]
    dt.a[v0:v1, :d] = _st(dt, acc)


# ---- matmul --------------------------------------------------------------------------------------------------------------
def _tile_dims(fl):
    return (256, 128) if fl & 64 else (128, 128) if fl & 32 else (64, 64)


def _matmul_region(b, a, m0, m1, n0, n1, A, B, exact):
    """Rows [m0,m1) x cols [n0,n1) of the tile: accumulate + epilogue in the reference's order (runtime/ref_gpt.py:69-103)."""
    out, bias, res, pre = b['out'], b['bias'], b['res'], b['pre']
    fl, K = a['flags'], a['K']
    ta, tb, accum, gelu, dg = fl & 1, fl & 2, fl & 4, fl & 8, fl & 512
    At = A[:K, m0:m1].T if ta else A[m0:m1, :K]
    Bt = B[n0:n1, :K].T if tb else B[:K, n0:n1]
    acc = _mm_seq(At, Bt) if exact else np.ascontiguousarray(At) @ np.ascontiguousarray(Bt)
    v = acc * f32(a['alpha'])
    if bias is not None:
        v = v + bias.flat[n0:n1]
    if dg:
        v = (v.astype(f64) * _gelu_grad(pre.a[m0:m1, n0:n1])).astype(np.float32)
    else:
        if pre is not None:
            pre.a[m0:m1, n0:n1] = _st(pre, v)
        if gelu:
            v = _gelu(v).astype(np.float32)
    if res is not None:
        v = v + res.a[m0:m1, n0:n1]
    if accum:
        v = out.a[m0:m1, n0:n1] + v
    out.a[m0:m1, n0:n1] = _st(out, v)


def _matmul_check(a, allowed):
    M, N, K, fl = a['M'], a['N'], a['K'], a['flags']
    _need(M > 0 and N > 0 and K > 0 and 0 <= a['m0'] < M and 0 <= a['n0'] < N, 'matmul_tile: bad M/N/K/m0/n0')
    _need(fl & ~allowed == 0 and not (fl & 32 and fl & 64) and not (fl & 256 and fl & 1024), f'matmul_tile: unsupported flags {fl}')


def matmul_tile(b, a, **kw):
    fl = a['flags']
    _matmul_check(a, 127 | 256 | 512 | 1024)
    if fl & 512:
        _need(b['pre'] is not None and b['bias'] is None and b['res'] is None and not fl & (4 | 8 | 128),
              'matmul_tile: flag 512 needs pre and refuses bias, res and flags 4, 8, 128')
    tm, tn = _tile_dims(fl)
    m1, n1 = min(a['m0'] + tm, a['M']), min(a['n0'] + tn, a['N'])
    _matmul_region(b, a, a['m0'], m1, a['n0'], n1, b['a'].a, b['b'].a, kw.get('exact_matmul', True))


def matmul_tile_bf16(b, a, **kw):
    """Operands rounded to bf16 on load, then matmul_tile (runtime/ref_extra.py:312-324)."""
    _matmul_check(a, 127 | 256 | 512 | 1024)
    tm, tn = _tile_dims(a['flags'])
    m1, n1 = min(a['m0'] + tm, a['M']), min(a['n0'] + tn, a['N'])
    A = b['a'].a if b['a'].dtype == BF16 else bf16_round(b['a'].a)
    B = b['b'].a if b['b'].dtype == BF16 else bf16_round(b['b'].a)
    _matmul_region(b, a, a['m0'], m1, a['n0'], n1, A, B, kw.get('exact_matmul', True))


def matmul_mma_bf16(b, a, **kw):
    """The 128 x 256 tile = eight 64 x 64 matmul_tile_bf16 tiles (runtime/ref_extra.py:326-331); done here as one region."""
    _matmul_check(a, 1 | 2 | 4 | 8)
    m1, n1 = min(a['m0'] + 128, a['M']), min(a['n0'] + 256, a['N'])
    A = b['a'].a if b['a'].dtype == BF16 else bf16_round(b['a'].a)
    B = b['b'].a if b['b'].dtype == BF16 else bf16_round(b['b'].a)
    _matmul_region(b, a, a['m0'], m1, a['n0'], n1, A, B, kw.get('exact_matmul', True))


# ---- normalisation ---------------------------------------------------------------------------------------------------------
def _norm_fwd(b, a, rms):
    x, g, out, rstd = b['x'], b['gamma'], b['out'], b['rstd']
    r0, r1, d = a['r0'], a['r1'], a['d']
    _need(0 <= r0 <= r1, 'norm_fwd: bad rows')
    row = x.a[r0:r1, :d].astype(f64)
    mu = np.zeros((r1 - r0, 1)) if rms else row.sum(axis=1, keepdims=True) / d
    rs = (1.0 / np.sqrt(((row - mu) ** 2).sum(axis=1, keepdims=True) / d + f64(f32(a['eps'])))).astype(np.float32)
    y = (row - mu) * rs.astype(f64) * g.flat[:d].astype(f64)
    if not rms:
        y = y + b['beta'].flat[:d].astype(f64)
    out.a[r0:r1, :d] = _st(out, y)
    rstd.flat[r0:r1] = rs[:, 0]
    if not rms:
        b['mean'].flat[r0:r1] = mu[:, 0].astype(np.float32)


def layernorm_fwd(b, a, **kw):
    _norm_fwd(b, a, False)


def rmsnorm_fwd(b, a, **kw):
    _norm_fwd(b, a, True)


def _norm_bwd_dx(b, a, rms):
    x, dy, g, rstd, dx = b['x'], b['dy'], b['gamma'], b['rstd'], b['dx']
    r0, r1, d = a['r0'], a['r1'], a['d']
    mu = np.zeros((r1 - r0, 1)) if rms else b['mean'].flat[r0:r1].astype(f64)[:, None]
    rs = rstd.flat[r0:r1].astype(f64)[:, None]
    gs = dy.a[r0:r1, :d].astype(f64) * g.flat[:d].astype(f64)
    xh = (x.a[r0:r1, :d].astype(f64) - mu) * rs
    s1 = np.zeros_like(mu) if rms else gs.sum(axis=1, keepdims=True) / d
    s2 = (gs * xh).sum(axis=1, keepdims=True) / d
    v = (rs * (gs - s1 - xh * s2)).astype(np.float32)
    if a['acc']:
        v = dx.a[r0:r1, :d] + v
    dx.a[r0:r1, :d] = _st(dx, v)


def layernorm_bwd_dx(b, a, **kw):
    _norm_bwd_dx(b, a, False)


def rmsnorm_bwd_dx(b, a, **kw):
    _norm_bwd_dx(b, a, True)


def norm_bwd_params(b, a, **kw):
    x, dy, mean, rstd, dg, db = b['x'], b['dy'], b['mean'], b['rstd'], b['dgamma'], b['dbeta']
    R, c0, c1 = a['R'], a['c0'], a['c1']
    _need(R >= 0 and 0 <= c0 <= c1 <= a['d'], 'norm_bwd_params: bad R/c0/c1/d')
    g = dy.a[:R, c0:c1].astype(f64)
    mu = mean.flat[:R].astype(f64)[:, None] if mean is not None else 0.0
    sg = (g * (x.a[:R, c0:c1].astype(f64) - mu) * rstd.flat[:R].astype(f64)[:, None]).sum(axis=0)
    sb = g.sum(axis=0)
    dg.flat[c0:c1] = _st(dg, (dg.flat[c0:c1].astype(f64) + sg) if a['acc'] else sg)
    if db is not None:
        db.flat[c0:c1] = _st(db, (db.flat[c0:c1].astype(f64) + sb) if a['acc'] else sb)


def colsum(b, a, **kw):
    x, out = b['x'], b['out']
    R, c0, c1 = a['R'], a['c0'], a['c1']
    s = np.zeros(c1 - c0, np.float32)
    xa = x.a
    for r in range(R):                       # s = f32(s + x[r,c]), rows ascending (runtime/ref_gpt.py:176-182)
        s += xa[r, c0:c1]
    out.flat[c0:c1] = _st(out, out.flat[c0:c1] + s if a['acc'] else s)


# ---- elementwise -----------------------------------------------------------------------------------------------------------
def gelu_fwd(b, a, **kw):
    e0, e1 = a['e0'], a['e1']
    b['out'].flat[e0:e1] = _st(b['out'], _gelu(b['x'].flat[e0:e1]))


def gelu_bwd(b, a, **kw):
    e0, e1 = a['e0'], a['e1']
    v = (b['dy'].flat[e0:e1].astype(f64) * _gelu_grad(b['x'].flat[e0:e1])).astype(np.float32)
    dx = b['dx']
    dx.flat[e0:e1] = _st(dx, dx.flat[e0:e1] + v if a['acc'] else v)


def residual_add(b, a, **kw):
    e0, e1 = a['e0'], a['e1']
    b['out'].flat[e0:e1] = _st(b['out'], b['a'].flat[e0:e1] + b['b'].flat[e0:e1])


def sgd_range(b, a, **kw):
    e0, e1 = a['e0'], a['e1']
    w = b['w'].flat
    w[e0:e1] = w[e0:e1] - f32(a['lr']) * b['g'].flat[e0:e1]


def round_tf32(b, a, **kw):
    e0, e1 = a['e0'], a['e1']
    b['out'].flat[e0:e1] = tf32_round(b['x'].flat[e0:e1])


def round_bf16(b, a, **kw):
    e0, e1 = a['e0'], a['e1']
    b['out'].flat[e0:e1] = bf16_round(b['x'].flat[e0:e1])


def zero_buf(b, a, **kw):
    b['x'].flat[a['e0']:a['e1']] = 0


def counter_inc(b, a, **kw):
    x = b['x'].flat
    x[a['i0']:a['i1']] = (x[a['i0']:a['i1']].astype(np.int64) + a['delta'] + 2**31) % 2**32 - 2**31


def scale_flat(b, a, **kw):
    e0, e1 = a['e0'], a['e1']
    b['out'].flat[e0:e1] = _st(b['out'], f32(a['alpha']) * b['x'].flat[e0:e1])


def add_rowtile(b, a, **kw):
    r0, r1, d = a['r0'], a['r1'], a['d']
    b['out'].a[r0:r1, :d] = _st(b['out'], b['x'].a[r0:r1, :d] + b['pos'].a[np.arange(r0, r1) % a['T'], :d])


_ACT = {0: (lambda x: np.where(x > 0, x, 0.0).astype(f64), lambda x: np.where(x > 0, 1.0, 0.0)),
        1: (_silu, _silu_d),
        2: (lambda x: np.tanh(x.astype(f64)), lambda x: 1.0 - np.tanh(x.astype(f64)) ** 2),
        3: (_sig, lambda x: _sig(x) * (1.0 - _sig(x)))}


def act_fwd(b, a, **kw):
    _need(a['kind'] in _ACT, 'act_fwd: kind not in 0..3')
    e0, e1 = a['e0'], a['e1']
    b['out'].flat[e0:e1] = _st(b['out'], _ACT[a['kind']][0](b['x'].flat[e0:e1]))


def act_bwd(b, a, **kw):
    _need(a['kind'] in _ACT, 'act_bwd: kind not in 0..3')
    e0, e1 = a['e0'], a['e1']
    v = (b['dy'].flat[e0:e1].astype(f64) * _ACT[a['kind']][1](b['x'].flat[e0:e1])).astype(np.float32)
    dx = b['dx']
    dx.flat[e0:e1] = _st(dx, dx.flat[e0:e1] + v if a['acc'] else v)


def silu_mul_fwd(b, a, **kw):
    e0, e1 = a['e0'], a['e1']
    b['out'].flat[e0:e1] = _st(b['out'], _silu(b['gate'].flat[e0:e1]) * b['up'].flat[e0:e1].astype(f64))


def _rope_rot(x1, x2, pos, i, hd, theta, sign):
    """Pairs (i, i+hd/2): ang = f32(f32(pos) * f32(theta^(-f32(2i)/hd))) (runtime/ref_gpt.py:250-262)."""
    inv = np.power(f64(f32(theta)), -(2.0 * i).astype(np.float32).astype(f64) / hd).astype(np.float32)
    ang = (pos.astype(np.float32)[:, None] * inv[None, :]).astype(np.float32).astype(f64)
    s, c = sign * np.sin(ang).astype(np.float32).astype(f64), np.cos(ang).astype(np.float32).astype(f64)
    x1, x2 = x1.astype(f64), x2.astype(f64)
    return (x1 * c - x2 * s).astype(np.float32), (x1 * s + x2 * c).astype(np.float32)


def _rope(b, a, sign):
    x, out, pos = b['x'], b['out'], b['pos']
    r0, r1, T, H, hd = a['r0'], a['r1'], a['T'], a['H'], a['hd']
    _need(T > 0 and H > 0 and hd > 0 and hd % 2 == 0, 'rope: bad T/H/hd')
    half = hd // 2
    p0 = int(pos.flat[0]) if pos is not None else 0
    p = (np.arange(r0, r1) % T + p0)
    i = np.arange(half)
    xa = x.a[r0:r1, :H * hd].reshape(r1 - r0, H, hd)
    res = np.empty_like(xa, dtype=np.float32)
    for h in range(H):
        y1, y2 = _rope_rot(xa[:, h, :half], xa[:, h, half:], p, i, hd, a['theta'], sign)
        res[:, h, :half], res[:, h, half:] = y1, y2
    out.a[r0:r1, :H * hd] = _st(out, res.reshape(r1 - r0, H * hd))


def rope_fwd(b, a, **kw):
    _rope(b, a, 1.0)


def rope_bwd(b, a, **kw):
    _rope(b, a, -1.0)


# ---- attention (training) ---------------------------------------------------------------------------------------------------
def _geom(a):
    _need(a['hd'] in (16, 32, 64, 128), 'attention: hd not in 16/32/64/128')
    _need(a['T'] > 0 and a['H'] > 0 and a['b'] >= 0, 'attention: bad T/H/b')


def attn_fwd(b, a, **kw):
    _geom(a)
    q, k, v, o, lse = b['q'], b['k'], b['v'], b['o'], b['lse']
    bb, h, T, H, Hkv, hd, sc = a['b'], a['h'], a['T'], a['H'], a['Hkv'], a['hd'], f64(f32(a['scale']))
    kvh = h // (H // Hkv)
    q0, q1 = a['q0'], min(a['q0'] + ATTN_ROWS, T)
    Q = q.a[bb * T + q0:bb * T + q1, h * hd:(h + 1) * hd].astype(f64)
    K = k.a[bb * T:bb * T + q1, kvh * hd:(kvh + 1) * hd].astype(f64)
    V = v.a[bb * T:bb * T + q1, kvh * hd:(kvh + 1) * hd].astype(f64)
    S = (Q @ K.T) * sc
    mask = np.arange(q1)[None, :] > np.arange(q0, q1)[:, None]
    S[mask] = -np.inf
    m = S.max(axis=1, keepdims=True)
    P = np.exp(S - m)
    l = P.sum(axis=1, keepdims=True)
    o.a[bb * T + q0:bb * T + q1, h * hd:(h + 1) * hd] = _st(o, (P @ V) / l)
    lse.flat[(bb * H + h) * T + q0:(bb * H + h) * T + q1] = (m + np.log(l))[:, 0].astype(np.float32)


def attn_bwd_delta(b, a, **kw):
    o, do, delta = b['o'], b['do'], b['delta']
    r0, r1, T, H, hd = a['r0'], a['r1'], a['T'], a['H'], a['hd']
    prod = (o.a[r0:r1, :H * hd].astype(f64) * do.a[r0:r1, :H * hd].astype(f64)).reshape(r1 - r0, H, hd).sum(axis=2)
    r = np.arange(r0, r1)
    for h in range(H):
        delta.flat[((r // T) * H + h) * T + r % T] = prod[:, h].astype(np.float32)


def attn_bwd_dq(b, a, **kw):
    _geom(a)
    q, k, v, do, lse, delta, dq = (b[n] for n in ('q', 'k', 'v', 'do', 'lse', 'delta', 'dq'))
    bb, h, T, H, Hkv, hd, sc = a['b'], a['h'], a['T'], a['H'], a['Hkv'], a['hd'], f64(f32(a['scale']))
    kvh = h // (H // Hkv)
    q0, q1 = a['q0'], min(a['q0'] + ATTN_ROWS, T)
    Q = q.a[bb * T + q0:bb * T + q1, h * hd:(h + 1) * hd].astype(f64)
    dO = do.a[bb * T + q0:bb * T + q1, h * hd:(h + 1) * hd].astype(f64)
    K = k.a[bb * T:bb * T + q1, kvh * hd:(kvh + 1) * hd].astype(f64)
    V = v.a[bb * T:bb * T + q1, kvh * hd:(kvh + 1) * hd].astype(f64)
    li = lse.flat[(bb * H + h) * T + q0:(bb * H + h) * T + q1].astype(f64)[:, None]
    di = delta.flat[(bb * H + h) * T + q0:(bb * H + h) * T + q1].astype(f64)[:, None]
    P = np.exp((Q @ K.T) * sc - li)
    P[np.arange(q1)[None, :] > np.arange(q0, q1)[:, None]] = 0.0
    dS = P * (dO @ V.T - di)
    dq.a[bb * T + q0:bb * T + q1, h * hd:(h + 1) * hd] = _st(dq, (dS @ K) * sc)


def attn_bwd_dkv(b, a, **kw):
    q, k, v, do, lse, delta, dk, dv = (b[n] for n in ('q', 'k', 'v', 'do', 'lse', 'delta', 'dk', 'dv'))
    bb, kvh, T, H, hd, sc = a['b'], a['kvh'], a['T'], a['H'], a['hd'], f64(f32(a['scale']))
    _need(hd in (16, 32, 64, 128) and T > 0 and H > 0 and bb >= 0 and kvh >= 0, 'attn_bwd_dkv: bad geometry')
    G = H // (k.cols // hd)
    k0, k1 = a['k0'], min(a['k0'] + ATTN_ROWS, T)
    K = k.a[bb * T + k0:bb * T + k1, kvh * hd:(kvh + 1) * hd].astype(f64)
    V = v.a[bb * T + k0:bb * T + k1, kvh * hd:(kvh + 1) * hd].astype(f64)
    sk, sv = np.zeros_like(K), np.zeros_like(V)
    mask = np.arange(k0, T)[:, None] < np.arange(k0, k1)[None, :]          # query before key: masked
    for h in range(kvh * G, (kvh + 1) * G):
        Q = q.a[bb * T + k0:bb * T + T, h * hd:(h + 1) * hd].astype(f64)
        dO = do.a[bb * T + k0:bb * T + T, h * hd:(h + 1) * hd].astype(f64)
        li = lse.flat[(bb * H + h) * T + k0:(bb * H + h) * T + T].astype(f64)[:, None]
        di = delta.flat[(bb * H + h) * T + k0:(bb * H + h) * T + T].astype(f64)[:, None]
        P = np.exp((Q @ K.T) * sc - li)
        P[mask] = 0.0
        sv += P.T @ dO
        sk += (P * (dO @ V.T - di)).T @ Q
    dk.a[bb * T + k0:bb * T + k1, kvh * hd:(kvh + 1) * hd] = _st(dk, sk * sc)
    dv.a[bb * T + k0:bb * T + k1, kvh * hd:(kvh + 1) * hd] = _st(dv, sv)


# ---- serving ------------------------------------------------------------------------------------------------------------------
def kv_append(b, a, **kw):
    kn, vn, kc, vc, lens = b['knew'], b['vnew'], b['kc'], b['vc'], b['lens']
    nn, Hkv, hd, Tmax = a['n_new'], a['Hkv'], a['hd'], a['Tmax']
    for bb in range(a['b0'], a['b1']):
        L = int(lens.flat[bb])
        _need(0 <= L and L + nn <= Tmax, f'kv_append: sequence {bb} length {L} + {nn} exceeds Tmax {Tmax}')
    for bb in range(a['b0'], a['b1']):
        L = int(lens.flat[bb])
        for h in range(Hkv):
            row = (bb * Hkv + h) * Tmax + L
            kc.a[row:row + nn, :hd] = _st(kc, kn.a[bb * nn:(bb + 1) * nn, h * hd:(h + 1) * hd])
            vc.a[row:row + nn, :hd] = _st(vc, vn.a[bb * nn:(bb + 1) * nn, h * hd:(h + 1) * hd])


def attn_decode(b, a, **kw):
    q, kc, vc, lens, o = b['q'], b['kc'], b['vc'], b['lens'], b['o']
    bb, h, H, Hkv, hd, Tmax = a['b'], a['h'], a['H'], a['Hkv'], a['hd'], a['Tmax']
    n = int(lens.flat[bb]) + 1
    _need(n >= 1 and n <= Tmax, f'attn_decode: sequence {bb} length exceeds Tmax {Tmax}')
    base = (bb * Hkv + h // (H // Hkv)) * Tmax
    s = (kc.a[base:base + n, :hd].astype(f64) @ q.a[bb, h * hd:(h + 1) * hd].astype(f64)) * f64(f32(a['scale']))
    p = np.exp(s - s.max())
    o.a[bb, h * hd:(h + 1) * hd] = _st(o, (p @ vc.a[base:base + n, :hd].astype(f64)) / p.sum())


def attn_decode_part(b, a, **kw):
    q, kc, vc, lens, part = b['q'], b['kc'], b['vc'], b['lens'], b['part']
    bb, kvh, s, S, H, Hkv, hd, Tmax, fl = (a[n] for n in ('b', 'kvh', 's', 'S', 'H', 'Hkv', 'hd', 'Tmax', 'flags'))
    _need(fl in (0, 1, 3) and 0 < hd <= 128 and hd % 8 == 0 and H // Hkv <= 8, 'attn_decode_part: bad flags/hd/group')
    p0 = int(lens.flat[bb])
    n = p0 + 1
    _need(p0 >= 0 and n <= Tmax, f'attn_decode_part: sequence {bb} length {p0} exceeds Tmax {Tmax}')
    chunk = -(-n // S)
    j0, j1 = s * chunk, min(n, s * chunk + chunk)
    G, base, half = H // Hkv, (bb * Hkv + kvh) * Tmax, hd // 2
    i = np.arange(half)
    pos = np.array([p0])
    if fl & 1 and j0 <= n - 1 < j1:
        kn, vn = b['knew'], b['vnew']
        y1, y2 = _rope_rot(kn.a[bb:bb + 1, kvh * hd:kvh * hd + half], kn.a[bb:bb + 1, kvh * hd + half:(kvh + 1) * hd], pos, i, hd, a['theta'], 1.0)
        kc.a[base + n - 1, :half], kc.a[base + n - 1, half:hd] = _st(kc, y1[0]), _st(kc, y2[0])
        vc.a[base + n - 1, :hd] = _st(vc, vn.a[bb, kvh * hd:(kvh + 1) * hd])
    for g in range(G):
        h = kvh * G + g
        qv = q.a[bb, h * hd:(h + 1) * hd].astype(np.float32)
        if fl & 1:
            y1, y2 = _rope_rot(qv[None, :half], qv[None, half:], pos, i, hd, a['theta'], 1.0)
            qv = np.concatenate([y1[0], y2[0]])
            if fl & 2:
                qv = bf16_round(qv)
        row = (bb * S + s) * H + h
        if j1 <= j0:
            part.a[row, :hd] = 0.0
            part.a[row, hd], part.a[row, hd + 1] = ATTN_EMPTY_M, 0.0
            continue
        sc = (kc.a[base + j0:base + j1, :hd].astype(f64) @ qv.astype(f64)) * f64(f32(a['scale']))
        m = sc.max()
        p = np.exp(sc - m)
        part.a[row, :hd] = (p @ vc.a[base + j0:base + j1, :hd].astype(f64)).astype(np.float32)
        part.a[row, hd], part.a[row, hd + 1] = f32(m), f32(p.sum())


def _rms_head(x, gamma, eps):
    """RMSNorm of one head vector, reference norm rounding (runtime/ref_gpt.py:107-173): statistics in double, rstd rounded to
    float32, out = f32(x * rs * gamma)."""
    ss = (x.astype(f64) ** 2).sum() / x.size
    rs = f32(1.0 / math.sqrt(ss + f64(f32(eps))))
    return (x.astype(f64) * f64(rs) * gamma.astype(f64)).astype(np.float32)


def attn_decode_part_qkn(b, a, **kw):
    """attn_decode_part with QK RMSNorm before the rotary embedding (an extension op, id 300): q heads and the appended key are
    normalised over the head dimension and scaled by qk_gamma rows 0 / 1; then exactly attn_decode_part on the normalised values."""
    bb, kvh, H, Hkv, hd = a['b'], a['kvh'], a['H'], a['Hkv'], a['hd']
    gam = b['qk_gamma']
    _need(gam.rows >= 2 and gam.cols >= hd, 'attn_decode_part_qkn: qk_gamma must be [2, hd]')
    G = H // Hkv
    q2 = Buf(b['q'].a.copy(), b['q'].dtype)
    for g in range(G):
        h = kvh * G + g
        q2.a[bb, h * hd:(h + 1) * hd] = _rms_head(b['q'].a[bb, h * hd:(h + 1) * hd], gam.a[0, :hd], a['eps'])
    b2 = dict(b, q=q2)
    if b.get('knew') is not None:
        k2 = Buf(b['knew'].a.copy(), b['knew'].dtype)
        k2.a[bb, kvh * hd:(kvh + 1) * hd] = _rms_head(b['knew'].a[bb, kvh * hd:(kvh + 1) * hd], gam.a[1, :hd], a['eps'])
        b2['knew'] = k2
    attn_decode_part(b2, a, **kw)


def attn_decode_merge(b, a, **kw):
    part, o = b['part'], b['o']
    bb, S, H, hd = a['b'], a['S'], a['H'], a['hd']
    for h in range(a['h0'], a['h1']):
        rows = np.array([(bb * S + s) * H + h for s in range(S)])
        live = rows[part.a[rows, hd + 1] > 0.0]
        M = part.a[live, hd].astype(f64).max()
        e = np.exp(part.a[live, hd].astype(f64) - M)
        L = (e * part.a[live, hd + 1].astype(f64)).sum()
        o.a[bb, h * hd:(h + 1) * hd] = _st(o, (e @ part.a[live, :hd].astype(f64)) / L)


def gemv_bf16(b, a, **kw):
    x, w, out, res = b['x'], b['w'], b['out'], b['res']
    K, pro, n0, n1 = a['K'], a['pro'], a['n0'], a['n1']
    _need(0 <= n0 < n1 and K > 0 and K % 8 == 0 and pro in (0, 1, 2), 'gemv_bf16: bad range, K or pro')
    xs = x.flat[:K].astype(f64)
    if pro == 1:
        rs = f64(f32(1.0 / math.sqrt((xs * xs).sum() / K + f64(f32(a['eps'])))))
        v = bf16_round((xs * rs * b['gamma'].flat[:K].astype(f64)).astype(np.float32))
    elif pro == 2:
        v = bf16_round((_silu(x.flat[:K]) * b['x2'].flat[:K].astype(f64)).astype(np.float32))
    else:
        v = bf16_round(x.flat[:K])
    y = w.a[n0:n1, :K].astype(f64) @ v.astype(f64)
    if res is not None:
        y = y + res.flat[n0:n1].astype(f64)
    out.flat[n0:n1] = _st(out, y)


def gemv_bf16_rows(b, a, **kw):
    """gemv_bf16 for rows r0..r1 of x / x2 / out / res against the same weight rows (an extension op, id 301): the batch of a
    decode step as rows of one activation matrix, so that the weights are read once for all of them.  Row by row it is exactly
    gemv_bf16 (same rounding points), which is how it is restated here."""
    r0, r1 = a['r0'], a['r1']
    _need(0 <= r0 < r1 and r1 <= b['x'].rows and r1 <= b['out'].rows, 'gemv_bf16_rows: bad row range')
    for r in range(r0, r1):
        row = {k: (None if v is None else (v if k in ('w', 'gamma') else Buf(v.a[r:r + 1], v.dtype))) for k, v in b.items()}
        gemv_bf16(row, a, **kw)


# ---- exchange between executors (extension ops 302 / 303) ---------------------------------------------------------------------------
# Restated from the reference's put_signal and inbox versions (include/mvm_ops_comm.def:5-11, include/mvm_dist.cuh:73-77, CPU
# model dist/commops.py): a peer buffer is simply another buffer of the table (in a CPU test: an array shared with the other
# rank's VM), the flag word is written after the data.  PEER_WAIT is how long peer_wait_sum polls before it gives up.
PEER_WAIT = 20.0


def _seq_ver(b, a):
    return a['ver'] + (int(b['seq'].a.flat[0]) * a['stride'] if b.get('seq') is not None else 0)


def peer_put_signal(b, a, **kw):
    n = a['n']
    _need(n > 0 and a['src_off'] >= 0 and a['src_off'] + n <= b['src'].a.size and a['dst_off'] >= 0 and a['dst_off'] + n <= b['dst'].a.size, 'peer_put_signal: range')
    _need(0 <= a['var'] < b['flag'].a.size, 'peer_put_signal: flag index')
    b['dst'].a.reshape(-1)[a['dst_off']:a['dst_off'] + n] = b['src'].a.reshape(-1)[a['src_off']:a['src_off'] + n]
    b['flag'].a.reshape(-1)[a['var']] = _seq_ver(b, a)          # after the data (release)


def peer_wait_sum(b, a, **kw):
    import time
    n, row0, rank, world = a['n'], a['row0'], a['rank'], a['world']
    _need(n > 0 and 1 <= world <= 32 and 0 <= rank < world and row0 >= 0, 'peer_wait_sum: arguments')
    _need(row0 + world <= b['flag'].a.size and row0 + world <= b['inbox'].rows and n <= b['inbox'].cols, 'peer_wait_sum: range')
    eff, flag = _seq_ver(b, a), b['flag'].a.reshape(-1)
    t0 = time.monotonic()
    while any(flag[row0 + p] < eff for p in range(world) if p != rank):
        _need(time.monotonic() - t0 < PEER_WAIT, 'peer_wait_sum: timeout')
        time.sleep(0.0005)
    po, oo = a.get('p_off', 0), a.get('o_off', 0)
    _need(po >= 0 and po + n <= b['partial'].a.size and oo >= 0 and oo + n <= b['out'].a.size, 'peer_wait_sum: offsets')
    v = None if b.get('res') is None else b['res'].a.reshape(-1)[:n].astype(np.float32)
    for p in range(world):
        t = (b['partial'].a.reshape(-1)[po:po + n] if p == rank else b['inbox'].a[row0 + p, :n]).astype(np.float32)
        v = t.copy() if v is None else (v + t).astype(np.float32)
    b['out'].a.reshape(-1)[oo:oo + n] = v


def peer_wait(b, a, **kw):
    import time
    row0, count = a['row0'], a['count']
    _need(row0 >= 0 and 1 <= count <= 32 and row0 + count <= b['flag'].a.size, 'peer_wait: range')
    eff, flag = _seq_ver(b, a), b['flag'].a.reshape(-1)
    t0 = time.monotonic()
    while any(flag[row0 + i] < eff for i in range(count)):
        _need(time.monotonic() - t0 < PEER_WAIT, 'peer_wait: timeout')
        time.sleep(0.0005)


# ---- loss -------------------------------------------------------------------------------------------------------------------
def softmax_ce_fwd(b, a, **kw):
    lg, tg, rl, ls = b['logits'], b['tgt'], b['rowloss'], b['lse']
    r0, r1, V, ign = a['r0'], a['r1'], a['V'], a['ignore']
    t = tg.flat[r0:r1]
    live = t != ign
    _need(((t[live] >= 0) & (t[live] < V)).all(), 'softmax_ce: target outside [0,V)')
    row = lg.a[r0:r1, :V].astype(f64)
    m = row.max(axis=1)
    lse = m + np.log(np.exp(row - m[:, None]).sum(axis=1))
    picked = row[np.arange(r1 - r0), np.where(live, t, 0)]
    ls.flat[r0:r1] = np.where(live, lse.astype(np.float32), f32(0))
    rl.flat[r0:r1] = np.where(live, (lse - picked).astype(np.float32), f32(0))


def softmax_ce_reduce(b, a, **kw):
    tg, rl, loss = b['tgt'], b['rowloss'], b['loss']
    live = tg.flat[:a['N']] != a['ignore']
    c = int(live.sum())
    s = float(rl.flat[:a['N']][live].astype(f64).sum())
    loss.flat[0] = f32(s / c) if c else f32(0)
    loss.flat[1] = f32(1.0 / c) if c else f32(0)


def softmax_ce_bwd(b, a, inv_count=None, **kw):
    lg, tg, ls, dl = b['logits'], b['tgt'], b['lse'], b['dlogits']
    r0, r1, V, ign = a['r0'], a['r1'], a['V'], a['ignore']
    f = f64(f32(f64(b['loss'].flat[1] if inv_count is None else inv_count) * f64(f32(a['scale']))))
    t = tg.flat[r0:r1]
    live = t != ign
    _need(((t[live] >= 0) & (t[live] < V)).all(), 'softmax_ce: target outside [0,V)')
    p = np.exp(lg.a[r0:r1, :V].astype(f64) - ls.flat[r0:r1].astype(f64)[:, None])
    p[np.arange(r1 - r0)[live], t[live]] -= 1.0
    p[~live] = 0.0
    dl.a[r0:r1, :V] = _st(dl, p * f)


def softmax_ce_fused(b, a, **kw):
    _need(a['ignore'] == -1 and a['N'] > 0, 'softmax_ce_fused: bad ignore/N')
    softmax_ce_fwd(b, a)
    softmax_ce_bwd(b, a, inv_count=f32(1.0 / a['N']))


# ---- optimiser ----------------------------------------------------------------------------------------------------------------
def _adamw(b, a, lr):
    p, g, m, v, gs, st = b['p'], b['g'], b['m'], b['v'], b['gscale'], b['step']
    t = int(st.flat[0])
    _need(t >= 1, f'adamw: step counter {t} < 1')
    b1, b2, eps, wd, lr = f32(a['b1']), f32(a['b2']), f32(a['eps']), f32(a['wd']), f32(lr)
    gsc = f32(gs.flat[0]) if gs is not None else f32(1.0)
    bc1 = f32(1.0 - f64(f32(math.pow(f64(b1), t))))
    bc2 = f32(1.0 - f64(f32(math.pow(f64(b2), t))))
    e0, e1 = a['e0'], a['e1']
    gi = g.flat[e0:e1].astype(np.float32) * gsc
    mi = b1 * m.flat[e0:e1] + f32(f64(1.0) - f64(b1)) * gi
    vi = b2 * v.flat[e0:e1] + (f32(f64(1.0) - f64(b2)) * gi) * gi
    m.flat[e0:e1], v.flat[e0:e1] = mi, vi
    pe = p.flat[e0:e1]
    decay = f32(f64(lr) * f64(wd)) * pe
    step = (lr * (mi / bc1)) / (np.sqrt(vi / bc2) + eps)
    p.flat[e0:e1] = (pe - decay) - step


def adamw(b, a, **kw):
    _adamw(b, a, a['lr'])


def adamw_lr(b, a, **kw):
    _adamw(b, a, b['lr'].flat[0])


def lr_schedule(b, a, **kw):
    t = int(b['step'].flat[0])
    warm = t / a['warmup'] if a['warmup'] > 0 and t <= a['warmup'] else 1.0
    prog = min(max((t - a['warmup']) / max(a['total'] - a['warmup'], 1), 0.0), 1.0)
    mr = float(f32(a['min_ratio']))
    f = {0: 1.0, 1: mr + (1 - mr) * 0.5 * (1 + math.cos(math.pi * prog)), 2: 1.0 - (1 - mr) * prog}[a['kind']]
    b['lr'].flat[0] = f32(float(f32(a['base'])) * warm * f)


def gradnorm_partial(b, a, **kw):
    g = b['g'].flat[a['e0']:a['e1']].astype(f64)
    b['partial'].flat[a['slot']] = f32((g * g).sum())


def gradnorm_finish(b, a, **kw):
    n = f32(math.sqrt(float(b['partial'].flat[:a['nslots']].astype(f64).sum())))
    mx = f32(a['max_norm'])
    b['out'].flat[0] = f32(min(1.0, float(f32(f64(mx) / f64(f32(f64(n) + f64(f32(1e-6)))))))) if mx > 0 else f32(1.0)
    b['out'].flat[1] = n


# ---- sampling -----------------------------------------------------------------------------------------------------------------
M32 = 0xFFFFFFFF


def philox4x32_10(c, key):
    """Philox-4x32-10 (Salmon et al. 2011) as the reference keys it (runtime/ref_gpt.py:488-500)."""
    c, key = list(c), list(key)
    for _ in range(10):
        p0, p1 = 0xD2511F53 * c[0], 0xCD9E8D57 * c[2]
        c = [(p1 >> 32) ^ c[1] ^ key[0], p1 & M32, (p0 >> 32) ^ c[3] ^ key[1], p0 & M32]
        key = [(key[0] + 0x9E3779B9) & M32, (key[1] + 0xBB67AE85) & M32]
    return c


def philox_uniform(seed, ctr, row):
    return (philox4x32_10([row & M32, ctr & M32, 0, 0], [seed & M32, 0x9E3779B9])[0] >> 8) * (1.0 / 16777216.0)


def _argmax_rows(x):
    return np.argmax(np.where(np.isnan(x), -np.inf, x), axis=1)


def argmax(b, a, **kw):
    r0, r1 = a['r0'], a['r1']
    b['out'].flat[r0:r1] = _argmax_rows(b['logits'].a[r0:r1, :a['V']])


def sample(b, a, **kw):
    lg, out, ctr, V = b['logits'], b['out'], b['ctr'], a['V']
    cv = int(ctr.flat[0]) if ctr is not None else 0
    temp = float(f32(a['temp']))
    for r in range(a['r0'], a['r1']):
        row = lg.a[r, :V]
        if temp <= 0:
            out.flat[r] = _argmax_rows(row[None, :])[0]
            continue
        ok = ~np.isnan(row)
        mx = row[ok].max() if ok.any() else -np.inf
        bits = row.view(np.uint32).astype(np.int64)
        key = np.where(bits >> 31, bits ^ M32, bits ^ 0x80000000)
        thr = 0
        if 0 < a['topk'] < V:
            thr = np.sort(key)[::-1][a['topk'] - 1]
        keep = ok & (key >= thr)
        w = np.where(keep, np.exp((row - f32(mx)).astype(np.float32).astype(f64) / temp), 0.0)
        total = 0.0
        for x in w:
            total += x
        target = philox_uniform(a['seed'], cv, r) * total
        run, pick, last = 0.0, -1, -1
        for j in range(V):
            if keep[j]:
                run += w[j]
                last = j
                if run > target:
                    pick = j
                    break
        out.flat[r] = pick if pick >= 0 else max(last, 0)


# ---- plumbing -----------------------------------------------------------------------------------------------------------------
def select_window(b, a, **kw):
    src, dst = b['src'], b['dst']
    base = int(b['step'].flat[0]) * a['stride'] + a['off']
    _need(base >= 0 and base + a['i1'] <= src.flat.size, 'select_window: window outside src')
    dst.flat[a['i0']:a['i1']] = src.flat[base + a['i0']:base + a['i1']]


def gather_rows(b, a, **kw):
    src, idx, dst = b['src'], b['idx'], b['dst']
    r0, r1, d = a['r0'], a['r1'], a['d']
    i = idx.flat[r0:r1]
    _need(((i >= 0) & (i < src.rows)).all(), 'gather_rows: row index out of range')
    dst.a[r0:r1, :d] = _st(dst, src.a[i, :d])


OPS = {n: f for n, f in list(globals().items()) if callable(f) and not n.startswith('_') and n[0].islower()
       and n not in ('bf16_round', 'tf32_round', 'philox4x32_10', 'philox_uniform', 'f32', 'f64')}
