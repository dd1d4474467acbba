"""GPU parity of the multi-MLP training graph (several independent classifiers in one launch) against the CPU oracle."""
import numpy as np
import pytest

from kvm_b200.workloads.mlp import build_mlps, preset
from tests.parity import compare, run_both

pytestmark = pytest.mark.gpu


def _counts_ok(ex, bundle):
    execs, observed = ex.task_counts()
    assert (execs == 1).all(), 'a task did not run exactly once'
    assert np.array_equal(observed, bundle.tasks['indegree']), 'observed predecessor completions != indegree'


def test_two_small_mlps_three_steps_exact(kvm_lib):
    c = preset('mlp_small')
    b = build_mlps(c, 3).to_bundle()
    ex, vm, res = run_both(b)
    assert res.done == res.admitted == len(b.tasks)
    _counts_ok(ex, b)
    compare(ex, vm, 2e-6)                       # float32 path, same accumulation order as the oracle
    for mi in range(len(c.widths)):
        for s in range(3):
            got, ref = ex.read_buffer(f'm{mi}.loss.{s}')[0, 0], vm.buffer(f'm{mi}.loss.{s}').a[0, 0]
            assert abs(got - ref) <= 1e-6 * abs(ref)
    ex.close()


def test_three_widths_momentum_two_steps(kvm_lib):
    """Widths 128 / 384 / 1024 of the eight-model configuration at its real batch and input size, two SGD-momentum steps."""
    c = preset('mlp8', widths=(128, 384, 1024))
    b = build_mlps(c, 2).to_bundle()
    ex, vm, res = run_both(b)
    _counts_ok(ex, b)
    compare(ex, vm, 1e-5)
    for mi in range(3):
        for s in range(2):
            got, ref = ex.read_buffer(f'm{mi}.loss.{s}')[0, 0], vm.buffer(f'm{mi}.loss.{s}').a[0, 0]
            assert abs(got - ref) <= 1e-3 * abs(ref)          # float32 loss tolerance of the path
    ex.close()


def test_eight_mlps_one_launch(kvm_lib):
    """All eight widths (128 ... 2048) in one executor launch: every task once, losses equal to the oracle's."""
    c = preset('mlp8')
    b = build_mlps(c, 1).to_bundle()
    ex, vm, res = run_both(b, exact_matmul=False)
    assert res.done == len(b.tasks)
    _counts_ok(ex, b)
    for mi in range(8):
        got, ref = ex.read_buffer(f'm{mi}.loss.0')[0, 0], vm.buffer(f'm{mi}.loss.0').a[0, 0]
        assert abs(got - ref) <= 1e-3 * abs(ref)
    compare(ex, vm, 1e-4)
    ex.close()
