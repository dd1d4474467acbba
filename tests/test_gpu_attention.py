"""GPU parity of causal attention forward / backward (SIMT form and the tcgen05 form for bf16 hd=64) against the CPU oracle."""
import numpy as np
import pytest

from kvm_b200.workloads.graph import Graph
from tests.parity import compare, run_both

pytestmark = pytest.mark.gpu


def attn_bundle(B, T, H, Hkv, hd, dt, seed=0):
    rng = np.random.default_rng(seed)
    g = Graph('attn')
    N = B * T
    for n, heads in (('q', H), ('k', Hkv), ('v', Hkv), ('do', H)):
        g.data(n, rng.standard_normal((N, heads * hd)).astype(np.float32), dt)
    for n, heads in (('o', H), ('dq', H), ('dk', Hkv), ('dv', Hkv)):
        g.buffer(n, N, heads * hd, dt)
    g.buffer('lse', B * H * T, 1), g.buffer('delta', B * H * T, 1)
    sc = hd ** -0.5
    for b in range(B):
        for h in range(H):
            for q0 in range(0, T, 128):
                g.task('attn_fwd', {'q': 'q', 'k': 'k', 'v': 'v', 'o': 'o', 'lse': 'lse', 'b': b, 'h': h, 'q0': q0, 'T': T, 'H': H, 'Hkv': Hkv, 'hd': hd, 'scale': sc},
                       ['q', 'k', 'v'], [('o', (b * T + q0, b * T + min(q0 + 128, T)), (h * hd, (h + 1) * hd)), ('lse', ((b * H + h) * T + q0, (b * H + h) * T + min(q0 + 128, T)))])
    g.task('attn_bwd_delta', {'o': 'o', 'do': 'do', 'delta': 'delta', 'r0': 0, 'r1': N, 'T': T, 'H': H, 'hd': hd}, ['o', 'do'], ['delta'])
    for b in range(B):
        for h in range(H):
            for q0 in range(0, T, 128):
                g.task('attn_bwd_dq', {'q': 'q', 'k': 'k', 'v': 'v', 'do': 'do', 'lse': 'lse', 'delta': 'delta', 'dq': 'dq', 'b': b, 'h': h, 'q0': q0, 'T': T, 'H': H,
                                       'Hkv': Hkv, 'hd': hd, 'scale': sc}, ['q', 'k', 'v', 'do', 'lse', 'delta'],
                       [('dq', (b * T + q0, b * T + min(q0 + 128, T)), (h * hd, (h + 1) * hd))])
        for kvh in range(Hkv):
            for k0 in range(0, T, 128):
                g.task('attn_bwd_dkv', {'q': 'q', 'k': 'k', 'v': 'v', 'do': 'do', 'lse': 'lse', 'delta': 'delta', 'dk': 'dk', 'dv': 'dv', 'b': b, 'kvh': kvh, 'k0': k0,
                                        'T': T, 'H': H, 'hd': hd, 'scale': sc}, ['q', 'k', 'v', 'do', 'lse', 'delta'],
                       [('dk', (b * T + k0, b * T + min(k0 + 128, T)), (kvh * hd, (kvh + 1) * hd)), ('dv', (b * T + k0, b * T + min(k0 + 128, T)), (kvh * hd, (kvh + 1) * hd))])
    return g.to_bundle()


@pytest.mark.parametrize('shape', [(1, 128, 1, 1), (2, 256, 2, 2), (1, 512, 4, 2), (2, 384, 2, 1)])
def test_attention_tc_bf16_hd64(kvm_lib, shape):
    B, T, H, Hkv = shape
    b = attn_bundle(B, T, H, Hkv, 64, 'bf16')
    ex, vm, res = run_both(b)
    n_attn = int(np.isin(b.tasks['op_id'], (45, 47, 48)).sum())
    assert ex.tc_task_count() == n_attn, 'bf16 hd=64 attention must be planned onto the tcgen05 path'
    # P and dS pass through bf16 on the tensor-core path and outputs are bf16: agreement to bf16 resolution
    compare(ex, vm, 1.5e-2, tols={'lse': 1e-5, 'delta': 1e-2})
    ex.close()


@pytest.mark.parametrize('case', [(1, 96, 2, 2, 32, 'f32'), (2, 160, 2, 1, 16, 'f32'), (1, 200, 2, 2, 64, 'f32'), (1, 130, 2, 2, 128, 'bf16'), (1, 100, 1, 1, 64, 'bf16')])
def test_attention_simt(kvm_lib, case):
    B, T, H, Hkv, hd, dt = case
    b = attn_bundle(B, T, H, Hkv, hd, dt)
    ex, vm, res = run_both(b)
    assert ex.tc_task_count() == 0
    compare(ex, vm, 2e-5 if dt == 'f32' else 6e-3)
    ex.close()
