"""Shared helpers of the GPU parity tests: run a bundle on the executor (through the C ABI) and on the CPU oracle, compare."""
import numpy as np

from kvm_b200.executor import Executor
from oracle.vm_np import VM


# The key-projection bias has an exactly zero gradient (softmax is invariant to a per-query constant added to every score),
# so its computed gradient is pure rounding noise, which AdamW then normalises to +-lr steps: no implementation agrees with
# another on these four buffers (the reference checks post-AdamW weights by float64 replay for the same reason,
# tests/gptdiff/golden_check.py:5-18).
NOISE_ONLY = ('attn.k.b',)


def run_both(bundle, exact_matmul=True, flags=0, runs=1, trace=False, workers=0):
    vm = VM(bundle, exact_matmul=exact_matmul)
    for _ in range(runs):
        vm.run()
        if runs > 1:
            vm = _rewind(vm)
    ex = Executor(trace=trace, flags=flags, workers=workers)
    ex.load(bundle)
    res = None
    for _ in range(runs):
        res = ex.run()
    return ex, vm, res


def _rewind(vm):
    """A VM that runs the same tasks again on the current buffers / versions (what kvm_rearm does on the device)."""
    nv = VM(vm.bundle, exact_matmul=vm.exact, buffers=vm.bufs)
    nv.versions = {k: 0 for k in vm.versions}
    return nv


def rel_err(got, ref):
    got, ref = got.astype(np.float64).ravel(), ref.astype(np.float64).ravel()
    den = np.sqrt((ref * ref).sum())
    return float(np.sqrt(((got - ref) ** 2).sum()) / den) if den > 0 else float(np.abs(got).max())


def compare(ex, vm, tol, skip=(), tols=None):
    """Every buffer of the bundle: int buffers exact, float buffers relative L2 <= tol (tols: per-name-prefix overrides).
    Returns {name: err} of the float buffers."""
    errs, bad = {}, []
    for spec, buf in zip(vm.bundle.buffers, vm.bufs):
        name = spec['name']
        if any(name.startswith(s) for s in skip) or any(t in name for t in NOISE_ONLY):
            continue
        got = ex.read_buffer(name)
        if spec['dtype'] == 1:
            if not np.array_equal(got, buf.a):
                bad.append((name, 'int mismatch'))
            continue
        e = rel_err(got, buf.a)
        errs[name] = e
        t = tol
        for k, v in (tols or {}).items():
            if name.startswith(k):
                t = v
        if not (e <= t):
            bad.append((name, e))
    assert not bad, f'{len(bad)} buffers differ from the oracle, worst first: {sorted(bad, key=lambda x: -x[1] if not isinstance(x[1], str) else -1)[:8]}'
    return errs


def vm_from_device(ex, bundle, **vm_kw):
    """An oracle VM whose initial buffers are read back from the device right after loading (before any run).  For large models:
    the device materialises seeded buffers in milliseconds (bit for bit what the host generator gives, which its own test pins),
    numpy takes a minute per 100 M elements."""
    from oracle.ops_np import Buf
    bufs = []
    for spec in bundle.buffers:
        a = ex.read_buffer(spec['name'])
        bufs.append(Buf(np.ascontiguousarray(a), spec['dtype']))
    return VM(bundle, buffers=bufs, **vm_kw)
