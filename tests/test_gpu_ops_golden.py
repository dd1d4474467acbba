"""Every registered op on the GPU, one task at a time, against the REFERENCE's stored outputs: the per-op fixtures of
tests/golden/ops_golden.npz were produced by the reference's own pure-Python CPU ops (tests/golden/make_golden.py) and
cover all registered ops but `noop` and `spin` with the edge arguments its tests use (row / column offsets, acc = 1,
ignore = -100, mod = T, ragged tiles, optional buffers absent).  Each case becomes a one-task bundle that goes through
kvm_submit / kvm_run like any other program.

Tolerances are the reference's own for its device ops (include/mvm_ops_gpt.cuh:24-28, relative to max |reference|):
exact for integer outputs and for the ops whose float32 step order is normative (copies, elementwise float32 arithmetic,
the float32 matmul tiles, AdamW / SGD, embeddings); 1e-5 for norms / column sums / GELU / RoPE / cross-entropy (float32
reduction trees against the reference's double sums); 2e-5 for attention and decode.  A bf16-stored output may differ by one
bf16 unit in the last place where the float32 value before rounding sits on a rounding boundary.

A second set runs the row / flat ops on bf16 STORAGE (inputs rounded to bf16, outputs stored as bf16) against the CPU
oracle, which tests/test_oracle_golden.py pins to the same fixtures.
"""
import json
from pathlib import Path

import numpy as np
import pytest

from kvm_b200 import abi
from kvm_b200.workloads.graph import Graph
from oracle import ops_np
from oracle.ops_np import Buf

pytestmark = pytest.mark.gpu

G = Path(__file__).resolve().parent / 'golden'
_npz = np.load(G / 'ops_golden.npz')
_index = json.loads(bytes(_npz['index']).decode())
DT = {'f32': 0, 'i32': 1, 'bf16': 2}

# float32 outputs that must equal the reference bit for bit
EXACT = {'copy', 'add', 'scale', 'relu', 'sgd', 'sgd_range', 'fill', 'matmul', 'residual_add', 'round_tf32', 'round_bf16', 'scale_flat', 'add_rowtile',
         'zero_buf', 'embedding_fwd', 'embedding_bwd', 'gather_rows', 'adamw', 'adamw_lr', 'predict', 'kv_append'}
TOL = {'attn_fwd': 2e-5, 'attn_bwd_delta': 2e-5, 'attn_bwd_dq': 2e-5, 'attn_bwd_dkv': 2e-5, 'attn_decode': 2e-5, 'attn_decode_part': 2e-5,
       'attn_decode_merge': 2e-5, 'gemv_bf16': 2e-5}
DEFAULT_TOL = 1e-5


def one_task_bundle(op, bufs, scal):
    g = Graph('case')
    args = dict(scal)
    for name, b in bufs.items():
        if b is None:
            args[name] = None
        else:
            arr, dt = b
            g.data(name, arr, dt)
            args[name] = name
    g.task(op, args)
    return g.to_bundle()


def check(op, name, got, ref, stored_bf16, exact):
    if ref.dtype == np.int32:
        assert np.array_equal(got, ref), f'{op}.{name}: integer output differs'
        return
    got, ref = got.astype(np.float32), ref.astype(np.float32)
    same = got.view(np.uint32) == ref.view(np.uint32)
    if same.all():
        return
    assert not exact, f'{op}.{name}: {int((~same).sum())} of {same.size} elements differ from the reference bit pattern (worst {np.abs(got - ref).max()})'
    scale = float(np.abs(ref).max()) or 1.0
    tol = TOL.get(op, DEFAULT_TOL)
    err = np.abs(got.astype(np.float64) - ref.astype(np.float64))
    if stored_bf16:      # one unit in the last place of the stored type, on the elements that differ
        ulp = np.spacing(np.abs(ref)).astype(np.float64) * 65536
        assert (err <= 1.001 * ulp + tol * scale).all(), f'{op}.{name}: bf16 output off by more than one ulp (worst {err.max()}, scale {scale})'
    else:
        assert err.max() <= tol * scale, f'{op}.{name}: max |diff| {err.max():.3e} > {tol} * max|ref| {scale:.3e}'


@pytest.mark.parametrize('ci', range(len(_index)), ids=[f"{i}:{c['op']}" for i, c in enumerate(_index)])
def test_op_against_reference_fixture(kvm_lib, ci):
    from kvm_b200.executor import Executor
    case = _index[ci]
    op = case['op']
    bufs = {n: (None if dt is None else (_npz[f'c{ci}.in.{n}'], dt)) for n, dt in case['bufs'].items()}
    spec = abi.load_ops()[op]
    scal = {a.name: (float(np.float32(case['scalars'][a.name])) if a.type == 'f32' else int(case['scalars'][a.name])) for a in spec.args if a.type != 'buf'}
    bundle = one_task_bundle(op, bufs, scal)
    with Executor() as ex:
        ex.load(bundle)
        res = ex.run()
        assert res.done == 1
        execs, observed = ex.task_counts()
        assert execs.tolist() == [1] and observed.tolist() == [0]
        exact = op in EXACT or (op in ('matmul_tile', 'matmul_tile_bf16', 'matmul_mma_bf16') and not (scal['flags'] & (8 | 512)))
        for n, dt in case['bufs'].items():
            if dt is not None:
                check(op, n, ex.read_buffer(n), _npz[f'c{ci}.out.{n}'], dt == 'bf16', exact and dt != 'bf16')


# ---- bf16 storage variants ------------------------------------------------------------------------------------------------------
# (op, buffers switched to bf16 storage): the activations, never the float32 parameters / statistics.
BF16_VARIANTS = [
    ('layernorm_fwd', ('x', 'out')), ('rmsnorm_fwd', ('x', 'out')), ('layernorm_bwd_dx', ('x', 'dy', 'dx')), ('rmsnorm_bwd_dx', ('x', 'dy', 'dx')),
    ('norm_bwd_params', ('x', 'dy')), ('colsum', ('x',)), ('gelu_fwd', ('x', 'out')), ('gelu_bwd', ('x', 'dy', 'dx')), ('residual_add', ('a', 'b', 'out')),
    ('round_bf16', ('out',)), ('scale_flat', ('x', 'out')), ('silu_mul_fwd', ('gate', 'up', 'out')), ('softmax_ce_fwd', ('logits',)),
    ('softmax_ce_bwd', ('logits', 'dlogits')), ('softmax_ce_fused', ('logits', 'dlogits')), ('embedding_fwd', ('out',)), ('gather_rows', ('src', 'dst')),
    ('rope_fwd', ('x', 'out')), ('rope_bwd', ('x', 'out')), ('attn_fwd', ('q', 'k', 'v', 'o')), ('attn_bwd_delta', ('o', 'do')),
    ('attn_bwd_dq', ('q', 'k', 'v', 'do', 'dq')), ('attn_bwd_dkv', ('q', 'k', 'v', 'do', 'dk', 'dv')), ('attn_decode', ('kc', 'vc')),
    ('argmax', ('logits',)), ('add_rowtile', ('x', 'out')),
]


def _bf16(a):
    return ops_np.bf16_round(np.ascontiguousarray(a, np.float32))


@pytest.mark.parametrize('op, as_bf16', BF16_VARIANTS, ids=[v[0] for v in BF16_VARIANTS])
def test_op_on_bf16_storage_against_oracle(kvm_lib, op, as_bf16):
    from kvm_b200.executor import Executor
    ci = next(i for i, c in enumerate(_index) if c['op'] == op)
    case = _index[ci]
    bufs = {}
    for n, dt in case['bufs'].items():
        if dt is None:
            bufs[n] = None
        elif n in as_bf16:
            assert dt == 'f32'
            bufs[n] = (_bf16(_npz[f'c{ci}.in.{n}']), 'bf16')
        else:
            bufs[n] = (_npz[f'c{ci}.in.{n}'].copy(), dt)
    spec = abi.load_ops()[op]
    scal = {a.name: (float(np.float32(case['scalars'][a.name])) if a.type == 'f32' else int(case['scalars'][a.name])) for a in spec.args if a.type != 'buf'}
    ref = {n: (None if b is None else Buf(b[0].copy(), DT[b[1]])) for n, b in bufs.items()}
    ops_np.OPS[op](ref, scal, exact_matmul=True)
    with Executor() as ex:
        ex.load(one_task_bundle(op, bufs, scal))
        assert ex.run().done == 1
        for n, b in bufs.items():
            if b is not None:
                check(op, n, ex.read_buffer(n), ref[n].a, b[1] == 'bf16', False)
