"""GPU parity of the GEMM tile ops: tcgen05 path (matmul_mma_bf16 on aligned bf16 operands), its SIMT fallback, and the
bit-exact float32 tile (matmul_tile), against the CPU oracle; all four transposition cases, every epilogue, ragged edges."""
import numpy as np
import pytest

from kvm_b200.workloads.graph import Graph
from tests.parity import compare, run_both

pytestmark = pytest.mark.gpu


def gemm_bundle(op, M, N, K, flags, a_dt='bf16', b_dt='bf16', out_dt='f32', bias=False, res=None, pre=None, alpha=1.0, seed=0):
    rng = np.random.default_rng(seed)
    g = Graph('gemm')
    ta, tb = flags & 1, flags & 2
    A = rng.standard_normal((K, M) if ta else (M, K)).astype(np.float32)
    B = rng.standard_normal((N, K) if tb else (K, N)).astype(np.float32)
    g.data('a', A, a_dt), g.data('b', B, b_dt)
    g.data('out', rng.standard_normal((M, N)).astype(np.float32), out_dt)
    if bias:
        g.data('bias', rng.standard_normal((1, N)).astype(np.float32))
    if res:
        g.data('res', rng.standard_normal((M, N)).astype(np.float32), res)
    if pre:
        g.data('pre', rng.standard_normal((M, N)).astype(np.float32), pre)
    tm, tn = (128, 256) if op == 'matmul_mma_bf16' else (256, 128) if flags & 64 else (128, 128) if flags & 32 else (64, 64)
    for m0 in range(0, M, tm):
        for n0 in range(0, N, tn):
            g.task(op, {'a': 'a', 'b': 'b', 'out': 'out', 'bias': 'bias' if bias else None, 'res': 'res' if res else None, 'pre': 'pre' if pre else None,
                        'm0': m0, 'n0': n0, 'M': M, 'N': N, 'K': K, 'flags': flags, 'alpha': alpha})
    return g.to_bundle()


@pytest.mark.parametrize('flags', [0, 1, 2, 3])
@pytest.mark.parametrize('shape', [(128, 256, 64), (256, 512, 192), (200, 328, 136), (384, 256, 1024)])
def test_tc_transposes(kvm_lib, flags, shape):
    M, N, K = shape
    b = gemm_bundle('matmul_mma_bf16', M, N, K, flags)
    ex, vm, res = run_both(b, exact_matmul=False)
    assert ex.tc_task_count() == len(b.tasks), 'aligned bf16 operands must be planned onto the tcgen05 path'
    compare(ex, vm, 2e-5)      # f32 accumulation of exact bf16 products: only the summation order differs
    ex.close()


@pytest.mark.parametrize('case', [
    dict(bias=True), dict(bias=True, flags=8, pre='bf16', out_dt='bf16'), dict(res='f32', bias=True), dict(flags=4), dict(flags=4 | 2, out_dt='bf16'),
    dict(out_dt='bf16', res='bf16', alpha=0.5), dict(flags=8 | 1, pre='f32', bias=True),
])
def test_tc_epilogues(kvm_lib, case):
    case = dict(case)
    flags = case.pop('flags', 0)
    b = gemm_bundle('matmul_mma_bf16', 256, 512, 128, flags, **case)
    ex, vm, res = run_both(b, exact_matmul=False)
    compare(ex, vm, 4e-3 if 'bf16' in (case.get('out_dt'), case.get('pre')) else 2e-5)
    ex.close()


@pytest.mark.parametrize('flags', [0, 1, 2, 3, 8])
def test_tc_stacked_tiles(kvm_lib, flags, monkeypatch):
    """KVM_CFG_PAIR_TILES: row-adjacent tiles of one product run stacked as 256 x 256 tiles (an odd tile row is left single);
    every task still counts as executed exactly once and the result equals the oracle's."""
    from kvm_b200.executor import CFG_PAIR_TILES
    monkeypatch.setenv('KVM_B200_PAIR_DEPTH', '0')        # stack whatever is ready, however short the queue
    M, N, K = 640, 512, 448
    b = gemm_bundle('matmul_mma_bf16', M, N, K, flags, bias=bool(flags & 8), res='f32' if flags & 8 else None)
    ex, vm, res = run_both(b, exact_matmul=False, flags=CFG_PAIR_TILES, trace=True, workers=1)      # one worker: it pops a tile and finds the partner still free
    assert res.done == len(b.tasks)
    execs, observed = ex.task_counts()
    assert (execs == 1).all()
    s, e, sm = ex.trace()
    import collections
    starts = collections.Counter(zip(s.tolist(), sm.tolist()))
    assert sum(1 for v in starts.values() if v == 2) >= 1, 'no pair of tiles was stacked'
    compare(ex, vm, 2e-5)
    ex.close()


def test_mma_fallback_is_bit_exact(kvm_lib):
    """f32 operands cannot take the TMA path: the SIMT fallback accumulates k-ascending like the CPU model, bit for bit."""
    b = gemm_bundle('matmul_mma_bf16', 130, 260, 72, 2, a_dt='f32', b_dt='f32', bias=True)
    ex, vm, res = run_both(b, exact_matmul=True)
    assert np.array_equal(ex.read_buffer('out').view(np.uint32), vm.buffer('out').a.view(np.uint32))
    ex.close()


@pytest.mark.parametrize('flags', [0, 1, 2, 3, 32, 64 | 2, 8, 4])
def test_matmul_tile_f32_bit_exact(kvm_lib, flags):
    b = gemm_bundle('matmul_tile', 150, 200, 96, flags, a_dt='f32', b_dt='f32', bias=True, res='f32', pre=None)
    ex, vm, res = run_both(b, exact_matmul=True)
    if flags & 8:
        compare(ex, vm, 1e-6)
    else:
        assert np.array_equal(ex.read_buffer('out').view(np.uint32), vm.buffer('out').a.view(np.uint32))
    ex.close()


def test_matmul_tile_dgelu(kvm_lib):
    b = gemm_bundle('matmul_tile', 64, 128, 32, 512, a_dt='f32', b_dt='f32', pre='f32')
    ex, vm, res = run_both(b)
    compare(ex, vm, 1e-5)
    ex.close()
