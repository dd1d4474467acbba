#!/usr/bin/env python3
"""Generate the golden fixtures of tests/golden/ from a checkout of the reference (Bobliuuu/kvm):

  python tests/golden/make_golden.py /path/to/reference

  ops_golden.npz        for every on-path op: seeded inputs and the outputs of the reference's own pure-Python CPU ops
                        (runtime/ref_ops.py OPS), called directly, at sizes its scalar loops finish in seconds
  vectors.json          known-answer vectors the reference's tests hold for this path: SplitMix64 draws
                        (tests/test_registries.py:176-180), seeded-buffer bit patterns (tests/gpu/initgen_vectors.txt), Philox
                        and token-sampling cases (tests/test_gpt_ref.py:55-57, tests/gpu_ops/sample_vectors.json)
  gpt_micro_golden.json this repo's gpt_micro 2-step training workload compiled by the reference compiler and run on the
                        reference CPU VM (runtime/workload_vm.py run_golden): hash of the compiled bundle bytes, losses,
                        final weights' checksums and a few whole buffers
  ref_gpt_tiny_f32/, ref_gpt_tiny_bf16s/
                        bundle DIRECTORIES written by the reference's own frontend and compiler (bench/vs_pytorch/gen.py --model
                        gpt_tiny --steps 1, f32 and bf16s storage: RoPE, biases, untied head) with the final state of the reference
                        CPU VM (--emit-golden) kept as golden.npz (golden.json is 3 MB of text per bundle; the tests write it back
                        out as JSON where a tool wants the file)
The fixtures are data; nothing here is imported by the product.
"""
import hashlib
import json
import subprocess
import sys
import tempfile
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
ROOT = HERE.parents[1]
if len(sys.argv) < 2:
    sys.exit('usage: make_golden.py /path/to/reference')
REF = Path(sys.argv[1])
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(REF / 'runtime'))

import ref_ops  # noqa: E402  (the reference)
from ref_types import Buf as RefBuf  # noqa: E402

from kvm_b200 import abi  # noqa: E402


def bf16(a):
    u = np.ascontiguousarray(a, np.float32).view(np.uint32)
    return ((u + np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1))) & np.uint32(0xFFFF0000)).view(np.float32)


def cases(rng):
    """(op, {buf: (array, dtype)}, {scalar: value}) at tiny sizes. dtype 'f32' | 'i32' | 'bf16'."""
    f = lambda *s: rng.standard_normal(s).astype(np.float32)
    B, T, H, Hkv, hd = 2, 8, 4, 2, 16
    N, d, V = B * T, 24, 40
    q, k, v = f(N, H * hd), f(N, Hkv * hd), f(N, Hkv * hd)
    ids = rng.integers(0, V, (N, 1)).astype(np.int32)
    z = lambda *s: np.zeros(s, np.float32)
    out = []
    A = lambda op, bufs, sc: out.append((op, bufs, sc))
    A('copy', {'src': (f(1, 20), 'f32'), 'dst': (z(1, 20), 'f32')}, {'n': 17})
    A('add', {'a': (f(1, 20), 'f32'), 'b': (f(1, 20), 'f32'), 'out': (z(1, 20), 'f32')}, {'n': 20})
    A('scale', {'x': (f(1, 20), 'f32'), 'out': (z(1, 20), 'f32')}, {'alpha': 0.37, 'n': 20})
    A('relu', {'x': (f(1, 20), 'f32'), 'out': (z(1, 20), 'f32')}, {'n': 20})
    A('sgd', {'w': (f(1, 20), 'f32'), 'g': (f(1, 20), 'f32')}, {'lr': 0.05, 'n': 20})
    A('predict', {'x': (f(1, 20), 'f32'), 'w': (f(1, 1), 'f32'), 'out': (z(1, 20), 'f32')}, {'n': 20})
    A('mse_grad', {'pred': (f(1, 20), 'f32'), 'target': (f(1, 20), 'f32'), 'x': (f(1, 20), 'f32'), 'loss': (z(1, 1), 'f32'), 'grad': (z(1, 1), 'f32')}, {'n': 20})
    A('matmul', {'a': (f(5, 7), 'f32'), 'b': (f(7, 6), 'f32'), 'out': (z(5, 6), 'f32')}, {'m': 5, 'n': 6, 'k': 7})
    A('fill', {'x': (z(1, 20), 'f32')}, {'value': 1.25, 'n': 13})
    A('embedding_fwd', {'ids': (ids, 'i32'), 'wte': (f(V, d), 'f32'), 'wpe': (f(T, d), 'f32'), 'out': (z(N, d), 'f32')}, {'r0': 2, 'r1': N, 'T': T, 'd': d})
    A('embedding_bwd', {'ids': (ids, 'i32'), 'dout': (f(N, d), 'f32'), 'dtab': (f(V, d), 'f32')}, {'N': N, 'mod': 0, 'v0': 3, 'v1': 30, 'd': d, 'acc': 1})
    A('embedding_bwd', {'ids': None, 'dout': (f(N, d), 'f32'), 'dtab': (z(T, d), 'f32')}, {'N': N, 'mod': T, 'v0': 0, 'v1': T, 'd': d, 'acc': 0})
    for fl in (0, 1, 2, 3, 8, 4, 32, 64 | 2):
        M_, N_, K_ = 70, 66, 9
        A('matmul_tile', {'a': (f(K_, M_) if fl & 1 else f(M_, K_), 'f32'), 'b': (f(N_, K_) if fl & 2 else f(K_, N_), 'f32'), 'out': (f(M_, N_), 'f32'),
                          'bias': (f(1, N_), 'f32'), 'res': (f(M_, N_), 'f32'), 'pre': (z(M_, N_), 'f32')},
          {'m0': 64 if not fl & 96 else 0, 'n0': 0, 'M': M_, 'N': N_, 'K': K_, 'flags': fl, 'alpha': 0.5})
    A('matmul_tile', {'a': (f(16, 9), 'f32'), 'b': (f(9, 12), 'f32'), 'out': (z(16, 12), 'f32'), 'bias': None, 'res': None, 'pre': (f(16, 12), 'f32')},
      {'m0': 0, 'n0': 0, 'M': 16, 'N': 12, 'K': 9, 'flags': 512, 'alpha': 1.0})
    A('matmul_tile_bf16', {'a': (f(20, 9), 'f32'), 'b': (f(9, 12), 'f32'), 'out': (z(20, 12), 'bf16'), 'bias': (f(1, 12), 'f32'), 'res': None, 'pre': (z(20, 12), 'bf16')},
      {'m0': 0, 'n0': 0, 'M': 20, 'N': 12, 'K': 9, 'flags': 8, 'alpha': 1.0})
    A('matmul_mma_bf16', {'a': (bf16(f(9, 130)), 'bf16'), 'b': (bf16(f(70, 9)), 'bf16'), 'out': (f(130, 70), 'f32'), 'bias': None, 'res': (f(130, 70), 'f32'), 'pre': None},
      {'m0': 128, 'n0': 0, 'M': 130, 'N': 70, 'K': 9, 'flags': 3 | 4, 'alpha': 2.0})
    A('layernorm_fwd', {'x': (f(N, d), 'f32'), 'gamma': (f(1, d), 'f32'), 'beta': (f(1, d), 'f32'), 'out': (z(N, d), 'f32'), 'mean': (z(N, 1), 'f32'), 'rstd': (z(N, 1), 'f32')},
      {'r0': 1, 'r1': N, 'd': d, 'eps': 1e-5})
    A('rmsnorm_fwd', {'x': (f(N, d), 'f32'), 'gamma': (f(1, d), 'f32'), 'out': (z(N, d), 'f32'), 'rstd': (z(N, 1), 'f32')}, {'r0': 0, 'r1': N, 'd': d, 'eps': 1e-6})
    mean, rstd = f(N, 1) * 0.1, np.abs(f(N, 1)) + 0.5
    A('layernorm_bwd_dx', {'x': (f(N, d), 'f32'), 'dy': (f(N, d), 'f32'), 'gamma': (f(1, d), 'f32'), 'mean': (mean, 'f32'), 'rstd': (rstd, 'f32'), 'dx': (f(N, d), 'f32')},
      {'r0': 0, 'r1': N, 'd': d, 'acc': 1})
    A('rmsnorm_bwd_dx', {'x': (f(N, d), 'f32'), 'dy': (f(N, d), 'f32'), 'gamma': (f(1, d), 'f32'), 'rstd': (rstd, 'f32'), 'dx': (z(N, d), 'f32')},
      {'r0': 0, 'r1': N, 'd': d, 'acc': 0})
    A('norm_bwd_params', {'x': (f(N, d), 'f32'), 'dy': (f(N, d), 'f32'), 'mean': (mean, 'f32'), 'rstd': (rstd, 'f32'), 'dgamma': (f(1, d), 'f32'), 'dbeta': (f(1, d), 'f32')},
      {'R': N, 'd': d, 'c0': 2, 'c1': d, 'acc': 1})
    A('colsum', {'x': (f(N, d), 'f32'), 'out': (f(1, d), 'f32')}, {'R': N, 'c0': 0, 'c1': d, 'acc': 1})
    A('gelu_fwd', {'x': (f(1, 50) * 3, 'f32'), 'out': (z(1, 50), 'f32')}, {'e0': 3, 'e1': 50})
    A('gelu_bwd', {'x': (f(1, 50) * 3, 'f32'), 'dy': (f(1, 50), 'f32'), 'dx': (f(1, 50), 'f32')}, {'e0': 0, 'e1': 50, 'acc': 1})
    A('residual_add', {'a': (f(1, 50), 'f32'), 'b': (f(1, 50), 'f32'), 'out': (z(1, 50), 'f32')}, {'e0': 0, 'e1': 50})
    A('sgd_range', {'w': (f(1, 50), 'f32'), 'g': (f(1, 50), 'f32')}, {'lr': 0.01, 'e0': 5, 'e1': 45})
    A('round_tf32', {'x': (f(1, 50), 'f32'), 'out': (z(1, 50), 'f32')}, {'e0': 0, 'e1': 50})
    A('round_bf16', {'x': (f(1, 50), 'f32'), 'out': (z(1, 50), 'f32')}, {'e0': 0, 'e1': 50})
    A('scale_flat', {'x': (f(1, 50), 'f32'), 'out': (z(1, 50), 'f32')}, {'alpha': 0.125, 'e0': 0, 'e1': 50})
    A('add_rowtile', {'x': (f(N, d), 'f32'), 'pos': (f(T, d), 'f32'), 'out': (z(N, d), 'f32')}, {'r0': 0, 'r1': N, 'T': T, 'd': d})
    for kind in range(4):
        A('act_fwd', {'x': (f(1, 50) * 2, 'f32'), 'out': (z(1, 50), 'f32')}, {'kind': kind, 'e0': 0, 'e1': 50})
        A('act_bwd', {'x': (f(1, 50) * 2, 'f32'), 'dy': (f(1, 50), 'f32'), 'dx': (f(1, 50), 'f32')}, {'kind': kind, 'e0': 0, 'e1': 50, 'acc': kind & 1})
    A('silu_mul_fwd', {'gate': (f(1, 50), 'f32'), 'up': (f(1, 50), 'f32'), 'out': (z(1, 50), 'f32')}, {'e0': 0, 'e1': 50})
    for op in ('rope_fwd', 'rope_bwd'):
        A(op, {'x': (q.copy(), 'f32'), 'out': (z(N, H * hd), 'f32'), 'pos': (np.array([[5]], np.int32), 'i32')}, {'r0': 0, 'r1': N, 'T': T, 'H': H, 'hd': hd, 'theta': 10000.0})
    sc = hd ** -0.5
    o, lse = z(N, H * hd), z(B * H * T, 1)
    A('attn_fwd', {'q': (q, 'f32'), 'k': (k, 'f32'), 'v': (v, 'f32'), 'o': (o, 'f32'), 'lse': (lse, 'f32')}, {'b': 1, 'h': 3, 'q0': 0, 'T': T, 'H': H, 'Hkv': Hkv, 'hd': hd, 'scale': sc})
    do_, lse_, dl_ = f(N, H * hd), f(B * H * T, 1) + 3.0, f(B * H * T, 1) * 0.1
    A('attn_bwd_delta', {'o': (f(N, H * hd), 'f32'), 'do': (do_, 'f32'), 'delta': (z(B * H * T, 1), 'f32')}, {'r0': 0, 'r1': N, 'T': T, 'H': H, 'hd': hd})
    A('attn_bwd_dq', {'q': (q, 'f32'), 'k': (k, 'f32'), 'v': (v, 'f32'), 'do': (do_, 'f32'), 'lse': (lse_, 'f32'), 'delta': (dl_, 'f32'), 'dq': (z(N, H * hd), 'f32')},
      {'b': 1, 'h': 2, 'q0': 0, 'T': T, 'H': H, 'Hkv': Hkv, 'hd': hd, 'scale': sc})
    A('attn_bwd_dkv', {'q': (q, 'f32'), 'k': (k, 'f32'), 'v': (v, 'f32'), 'do': (do_, 'f32'), 'lse': (lse_, 'f32'), 'delta': (dl_, 'f32'), 'dk': (z(N, Hkv * hd), 'f32'),
                       'dv': (z(N, Hkv * hd), 'f32')}, {'b': 0, 'kvh': 1, 'k0': 0, 'T': T, 'H': H, 'hd': hd, 'scale': sc})
    Tmax = 12
    lens = np.array([[5], [7]], np.int32)
    kc, vc = f(B * Hkv * Tmax, hd), f(B * Hkv * Tmax, hd)
    A('kv_append', {'knew': (f(B * 2, Hkv * hd), 'f32'), 'vnew': (f(B * 2, Hkv * hd), 'f32'), 'kc': (kc.copy(), 'f32'), 'vc': (vc.copy(), 'f32'), 'lens': (lens, 'i32')},
      {'b0': 0, 'b1': B, 'n_new': 2, 'Hkv': Hkv, 'hd': hd, 'Tmax': Tmax})
    A('attn_decode', {'q': (f(B, H * hd), 'f32'), 'kc': (kc, 'f32'), 'vc': (vc, 'f32'), 'lens': (lens, 'i32'), 'o': (z(B, H * hd), 'f32')},
      {'b': 1, 'h': 3, 'H': H, 'Hkv': Hkv, 'hd': hd, 'Tmax': Tmax, 'scale': sc})
    S = 3
    for fl, s in ((0, 0), (0, 2), (1, 2), (3, 1), (3, 2)):
        A('attn_decode_part', {'q': (f(B, H * hd), 'f32'), 'kc': (bf16(kc), 'bf16'), 'vc': (bf16(vc), 'bf16'), 'lens': (lens, 'i32'), 'part': (z(B * S * H, hd + 2), 'f32'),
                               'knew': (f(B, Hkv * hd), 'f32') if fl else None, 'vnew': (f(B, Hkv * hd), 'f32') if fl else None},
          {'b': 1, 'kvh': 1, 's': s, 'S': S, 'H': H, 'Hkv': Hkv, 'hd': hd, 'Tmax': Tmax, 'scale': sc, 'theta': 1e6, 'flags': fl})
    part = f(B * S * H, hd + 2)
    part[:, hd + 1] = np.abs(part[:, hd + 1]) + 0.1
    part[(1 * S + 1) * H + 2, hd + 1] = 0.0
    A('attn_decode_merge', {'part': (part, 'f32'), 'o': (z(B, H * hd), 'bf16')}, {'b': 1, 'h0': 1, 'h1': 4, 'S': S, 'H': H, 'hd': hd})
    K = 32
    for pro in (0, 1, 2):
        A('gemv_bf16', {'x': (f(1, K), 'f32'), 'x2': (f(1, K), 'f32') if pro == 2 else None, 'gamma': (f(1, K), 'f32') if pro == 1 else None, 'w': (bf16(f(20, K)), 'bf16'),
                        'out': (z(1, 20), 'bf16' if pro == 2 else 'f32'), 'res': (f(1, 20), 'f32') if pro else None}, {'n0': 3, 'n1': 19, 'K': K, 'pro': pro, 'eps': 1e-6})
    logits, tgt = f(N, V) * 2, rng.integers(0, V, (N, 1)).astype(np.int32)
    tgt2 = tgt.copy()
    tgt2[3] = -100
    A('softmax_ce_fwd', {'logits': (logits, 'f32'), 'tgt': (tgt2, 'i32'), 'rowloss': (z(N, 1), 'f32'), 'lse': (z(N, 1), 'f32')}, {'r0': 0, 'r1': N, 'V': V, 'ignore': -100})
    A('softmax_ce_reduce', {'rowloss': (np.abs(f(N, 1)), 'f32'), 'tgt': (tgt2, 'i32'), 'loss': (z(1, 2), 'f32')}, {'N': N, 'ignore': -100})
    A('softmax_ce_bwd', {'logits': (logits, 'f32'), 'tgt': (tgt2, 'i32'), 'lse': (f(N, 1) + 4, 'f32'), 'loss': (np.array([[2.0, 1 / 15]], np.float32), 'f32'), 'dlogits': (z(N, V), 'f32')},
      {'r0': 0, 'r1': N, 'V': V, 'ignore': -100, 'scale': 0.5})
    A('softmax_ce_fused', {'logits': (logits, 'f32'), 'tgt': (tgt, 'i32'), 'rowloss': (z(N, 1), 'f32'), 'lse': (z(N, 1), 'f32'), 'dlogits': (z(N, V), 'f32')},
      {'r0': 0, 'r1': N, 'V': V, 'ignore': -1, 'N': N, 'scale': 1.0})
    step = np.array([[3]], np.int32)
    for op, extra_b, extra_s in (('adamw', {}, {'lr': 3e-4}), ('adamw_lr', {'lr': (np.array([[1e-3]], np.float32), 'f32')}, {})):
        A(op, {'p': (f(1, 50), 'f32'), 'g': (f(1, 50), 'f32'), 'm': (f(1, 50) * 0.1, 'f32'), 'v': (np.abs(f(1, 50)) * 0.01, 'f32'), 'gscale': (np.array([[0.7, 0]], np.float32), 'f32'),
               'step': (step, 'i32'), **extra_b}, {'e0': 2, 'e1': 50, 'b1': 0.9, 'b2': 0.999, 'eps': 1e-8, 'wd': 0.01, **extra_s})
    for kind in range(3):
        A('lr_schedule', {'step': (np.array([[7]], np.int32), 'i32'), 'lr': (z(1, 1), 'f32')}, {'kind': kind, 'base': 6e-4, 'warmup': 4, 'total': 20, 'min_ratio': 0.1})
    A('gradnorm_partial', {'g': (f(1, 50), 'f32'), 'partial': (z(1, 4), 'f32')}, {'slot': 2, 'e0': 0, 'e1': 50})
    A('gradnorm_finish', {'partial': (np.abs(f(1, 4)), 'f32'), 'out': (z(1, 2), 'f32')}, {'nslots': 4, 'max_norm': 1.0})
    A('argmax', {'logits': (logits, 'f32'), 'out': (np.zeros((N, 1), np.int32), 'i32')}, {'r0': 0, 'r1': N, 'V': V})
    A('sample', {'logits': (logits, 'f32'), 'out': (np.zeros((N, 1), np.int32), 'i32'), 'ctr': (np.array([[9]], np.int32), 'i32')},
      {'r0': 0, 'r1': N, 'V': V, 'temp': 0.8, 'topk': 5, 'seed': 1234})
    A('zero_buf', {'x': (f(1, 50), 'f32')}, {'e0': 5, 'e1': 20})
    A('counter_inc', {'x': (np.array([[1, 2147483647, 5]], np.int32), 'i32')}, {'i0': 0, 'i1': 2, 'delta': 1})
    A('select_window', {'src': (rng.integers(0, 99, (40, 1)).astype(np.int32), 'i32'), 'step': (np.array([[2]], np.int32), 'i32'), 'dst': (np.zeros((8, 1), np.int32), 'i32')},
      {'i0': 0, 'i1': 8, 'stride': 10, 'off': 1})
    A('gather_rows', {'src': (f(V, d), 'f32'), 'idx': (ids, 'i32'), 'dst': (z(N, d), 'f32')}, {'r0': 0, 'r1': N, 'd': d})
    return out


def run_reference_op(op, bufs, scal):
    ref = ref_ops.OPS[op]
    rb = {}
    for name, b in bufs.items():
        if b is None:
            rb[name] = None
            continue
        a, dt = b
        vals = [int(x) for x in a.reshape(-1)] if dt == 'i32' else [float(x) for x in a.reshape(-1)]
        rb[name] = RefBuf(vals, a.shape[0], a.shape[1], dt)
    sc = {}
    spec = abi.load_ops()[op]
    for arg in spec.args:
        if arg.type == 'f32':
            sc[arg.name] = float(np.float32(scal[arg.name]))
        elif arg.type == 'i32':
            sc[arg.name] = int(scal[arg.name])
    ref.run(rb, sc)
    return {n: np.array(list(b), dtype=np.int32 if b.dtype == 'i32' else np.float32).reshape(b.rows, b.cols) for n, b in rb.items() if b is not None}


def main():
    rng = np.random.default_rng(2026)
    store, index = {}, []
    for ci, (op, bufs, scal) in enumerate(cases(rng)):
        outs = run_reference_op(op, bufs, scal)
        index.append({'op': op, 'scalars': scal, 'bufs': {n: (None if b is None else b[1]) for n, b in bufs.items()}})
        for n, b in bufs.items():
            if b is not None:
                store[f'c{ci}.in.{n}'] = b[0]
                store[f'c{ci}.out.{n}'] = outs[n]
    store['index'] = np.frombuffer(json.dumps(index).encode(), dtype=np.uint8)
    np.savez_compressed(HERE / 'ops_golden.npz', **store)
    print('ops_golden.npz:', len(index), 'cases')

    # ---- known-answer vectors held by the reference's tests
    import initgen
    import ref_gpt
    vec = {'splitmix64_seed0': [initgen.draw(0, j) for j in range(3)], 'initgen': [], 'philox_kat': [], 'sample_cases': []}
    lines = (REF / 'tests/gpu/initgen_vectors.txt').read_text().split('\n')
    for head, body in zip(lines[0::2], lines[1::2]):
        if head.strip():
            seed, draws, bias, coef, n = head.split()
            vec['initgen'].append({'seed': int(seed), 'draws': int(draws), 'bias_bits': bias, 'coef_bits': coef, 'n': int(n), 'bits': body.split()})
    sv = json.loads((REF / 'tests/gpu_ops/sample_vectors.json').read_text())
    vec['philox_kat'] = sv['philox_kat'] + [{'counter': [0, 0, 0, 0], 'key': [0, 0], 'out': ref_gpt.philox4x32_10([0, 0, 0, 0], [0, 0])}]
    vec['sample_cases'] = sv['cases']
    (HERE / 'vectors.json').write_text(json.dumps(vec))
    print('vectors.json:', len(vec['initgen']), 'initgen,', len(vec['sample_cases']), 'sample cases')

    # ---- gpt_micro through the reference compiler and CPU VM
    from kvm_b200.workloads.gpt import build_training, preset
    g = build_training(preset('gpt_micro'), 2)
    with tempfile.TemporaryDirectory() as td:
        td = Path(td)
        (td / 'workload.json').write_text(json.dumps(g.to_spec()))
        subprocess.run([sys.executable, str(REF / 'runtime/compile_workload.py'), str(td / 'workload.json'), str(td / 'bundle'), '--emit-golden'], check=True,
                       capture_output=True)
        gold = json.loads((td / 'bundle/golden.json').read_text())
        sha = {n: hashlib.sha256((td / 'bundle' / n).read_bytes()).hexdigest() for n in ('tasks.bin', 'successors.bin', 'args.bin')}
    keep = ('loss.0', 'loss.1', 'clip_coef', 'w.lnf.g', 'w.h0.attn.q.b', 'g.h0.ln1.g')
    sums = {n: hashlib.sha256(np.array(v, np.float32 if gold['dtypes'][n] != 'i32' else np.int32).tobytes()).hexdigest() for n, v in gold['buffers'].items()}
    (HERE / 'gpt_micro_golden.json').write_text(json.dumps({'bundle_sha256': sha, 'versions': gold['versions'], 'buffers': {n: gold['buffers'][n] for n in keep},
                                                            'buffer_sha256': sums}))
    print('gpt_micro_golden.json: losses', gold['buffers']['loss.0'][0], gold['buffers']['loss.1'][0])

    # ---- bundle directories of the reference's own frontend (its gpt_tiny: RoPE, biases, untied head), f32 and bf16s storage
    import shutil
    for tag, extra in (('f32', []), ('bf16s', ['--precision', 'bf16s'])):
        with tempfile.TemporaryDirectory() as td:
            td = Path(td)
            subprocess.run([sys.executable, str(REF / 'bench/vs_pytorch/gen.py'), str(td / 'w'), '--model', 'gpt_tiny', '--steps', '1', *extra], check=True, capture_output=True)
            subprocess.run([sys.executable, str(REF / 'runtime/compile_workload.py'), str(td / 'w/workload.json'), str(td / 'b'), '--emit-golden'], check=True,
                           capture_output=True)
            out = HERE / f'ref_gpt_tiny_{tag}'
            shutil.rmtree(out, ignore_errors=True)
            out.mkdir()
            for n in ('tasks.bin', 'successors.bin', 'args.bin', 'metadata.json'):
                shutil.copy(td / 'b' / n, out / n)
            meta = json.loads((td / 'b/metadata.json').read_text())
            for b in meta['buffers']:                      # `file` inits travel with the bundle
                if b['init']['kind'] == 'file':
                    (out / b['init']['path']).parent.mkdir(parents=True, exist_ok=True)
                    shutil.copy(td / 'b' / b['init']['path'], out / b['init']['path'])
            gold = json.loads((td / 'b/golden.json').read_text())
            arrs = {'buf.' + n: np.array(v, np.int32 if gold['dtypes'][n] == 'i32' else np.float32) for n, v in gold['buffers'].items()}
            arrs['meta'] = np.frombuffer(json.dumps({'versions': gold['versions'], 'dtypes': gold['dtypes']}).encode(), dtype=np.uint8)
            np.savez_compressed(out / 'golden.npz', **arrs)
            print(f'ref_gpt_tiny_{tag}:', meta['task_count'], 'tasks, loss', gold['buffers']['loss.0'][0])


if __name__ == '__main__':
    main()
