"""Parity at the shapes the benchmark times, and the acceptance criteria as the task states them.

  * GPT-162M tiles (d 768, 12 heads of 64, FFN 3072, vocabulary 50304 with its ragged last 128 x 256 tile, T 1024): one training
    step of the 2-layer / micro-batch-4 cut `gpt_162m_2l` against the CPU oracle: bf16 loss within 1e-2 relative, every buffer
    within a stated relative L2.
  * Qwen3-8B decode tiles (hidden 4096, 32 query / 8 kv heads of 128, FFN 12288, context 4096): 32 greedy tokens of the 4-layer
    cut identical to the oracle's (vocabulary cut to 32768 so the float32 CPU copy of the weights stays at 4 GB).
  * Configuration 1 as stated: the tiny GPT, 20 AdamW steps, float32: the loss of EVERY step within 1e-3 relative of the
    oracle's, and the final weights no further from an all-double rerun (oracle/f64.py) than twice the float32 oracle is.
"""
import numpy as np
import pytest

from tests.parity import NOISE_ONLY, rel_err, vm_from_device

pytestmark = pytest.mark.gpu

# Weight seed of the decode test.  Greedy decoding compares arg-max tokens, so a step where the two largest logits of the CPU
# model are closer than the rounding noise between two float32 summation orders (about 1e-3 of the logits' spread at this depth)
# can go either way on ANY implementation.  With seed 0 that happens at step 24 (gap 0.00056 at a spread of 1.28: the device takes
# the runner-up and every later token differs); with seed 1 the smallest top-2 gap over the 32 steps is 0.021.
SEED = 1


def test_gpt_162m_shapes_one_step(kvm_lib):
    from kvm_b200.executor import Executor
    from kvm_b200.workloads.gpt import build_training, preset
    cfg = preset('gpt_162m_2l')
    b = build_training(cfg, 1).to_bundle(check=False)
    with Executor() as ex:
        ex.load(b)
        assert ex.tc_task_count() > 0.6 * len(b.tasks), 'the GEMM tiles and attention blocks of this shape must take the tcgen05 path'
        vm = vm_from_device(ex, b, exact_matmul=False)
        res = ex.run()
        assert res.done == len(b.tasks)
        execs, observed = ex.task_counts()
        assert (execs == 1).all() and np.array_equal(observed, b.tasks['indegree'])
        vm.run()
        got, ref = float(ex.read_buffer('loss.0')[0, 0]), float(vm.buffer('loss.0').a[0, 0])
        assert abs(got - ref) <= 1e-2 * abs(ref), (got, ref)            # the stated bf16 tolerance
        assert abs(got - ref) <= 2e-4 * abs(ref), (got, ref)            # what this path actually holds
        # Activations and gradients stored as bf16 differ by a bf16 ulp wherever the float32 value before rounding sits on a
        # boundary, and those differences travel on through the layers: 2e-2 relative L2.  Float32 buffers that are sums of many
        # such values (weight gradients, the post-AdamW state) 2e-2 as well.  Integers exact.
        bad, worst = [], {}
        for spec, buf in zip(b.buffers, vm.bufs):
            name = spec['name']
            if any(t in name for t in NOISE_ONLY):
                continue
            if name.startswith('w.') and name.endswith('.b'):
                # Biases start at zero: after this first AdamW step they are -lr * g / (|g| + eps), i.e. lr * sign(g) wherever |g| >> eps.
                # A gradient element at the noise level of the bf16 activations may have either sign, and the whole value flips with
                # it (0.1% of the elements here: 7% relative L2).  Their gradients g.* and moments m.* / v.* are compared below like
                # every other buffer; the reference judges post-AdamW weights by a float64 replay for the same reason
                # (tests/gptdiff/golden_check.py:5-18).
                continue
            g = ex.read_buffer(name)
            if spec['dtype'] == 1:
                if not np.array_equal(g, buf.a):
                    bad.append((name, 'int'))
                continue
            e = rel_err(g, buf.a)
            worst[name] = e
            if not e <= 2e-2:
                bad.append((name, e))
        assert not bad, f'{len(bad)} buffers beyond tolerance, e.g. {sorted(bad, key=lambda x: -x[1] if not isinstance(x[1], str) else 0)[:8]}'


def test_qwen3_8b_shapes_32_greedy_tokens(kvm_lib):
    from kvm_b200.executor import Executor
    from kvm_b200.workloads.decode import build_decode, preset
    from oracle.vm_np import VM
    cfg = preset('qwen3_8b_4l', vocab=32768, seed=SEED)
    b = build_decode(cfg).to_bundle(check=False)
    got, ref = [], []
    with Executor() as ex:
        ex.load(b)
        vm = vm_from_device(ex, b, exact_matmul=False)
        for s in range(32):
            res = ex.run()
            assert res.done == len(b.tasks)
            got.append(int(ex.read_buffer('u0.tok')[0, 0]))
        execs, observed = ex.task_counts()
        assert (execs == 1).all() and np.array_equal(observed, b.tasks['indegree'])
        assert int(ex.read_buffer('u0.lens')[0, 0]) == cfg.ctx + 32
    for s in range(32):
        vm.run()
        ref.append(int(vm.buffer('u0.tok').a[0, 0]))
        vm = VM(b, exact_matmul=False, buffers=vm.bufs)
    assert got == ref, f'first difference at step {next(i for i in range(32) if got[i] != ref[i])}: {got} vs {ref}'
    assert len(set(ref)) > 4, 'degenerate test: the model keeps emitting the same tokens'


def test_tiny_gpt_20_steps_loss_and_f64_deviation(kvm_lib):
    from kvm_b200.executor import Executor
    from kvm_b200.workloads.gpt import build_training, preset
    from oracle.vm_np import VM
    steps = 20
    b = build_training(preset('gpt_tiny'), steps).to_bundle()
    v32 = VM(b, exact_matmul=False).run()
    v64 = VM(b, exact_matmul=False, f64=True).run()
    with Executor() as ex:
        ex.load(b)
        res = ex.run()
        assert res.done == len(b.tasks)
        execs, observed = ex.task_counts()
        assert (execs == 1).all() and np.array_equal(observed, b.tasks['indegree'])
        for s in range(steps):
            got, ref = float(ex.read_buffer(f'loss.{s}')[0, 0]), float(v32.buffer(f'loss.{s}').a[0, 0])
            assert abs(got - ref) <= 1e-3 * abs(ref), (s, got, ref)
        num_g = num_r = 0.0
        bad = []
        for spec, r32, r64 in zip(b.buffers, v32.bufs, v64.bufs):
            name = spec['name']
            if not name.startswith('w.'):
                continue
            dg = ex.read_buffer(name).astype(np.float64) - r64.a
            dr = r32.a.astype(np.float64) - r64.a
            num_g += float((dg * dg).sum()); num_r += float((dr * dr).sum())
            if not any(t in name for t in NOISE_ONLY) and not np.sqrt((dg * dg).sum()) <= 2.0 * np.sqrt((dr * dr).sum()) + 1e-9:
                bad.append((name, float(np.sqrt((dg * dg).sum())), float(np.sqrt((dr * dr).sum()))))
        assert np.sqrt(num_g) <= 2.0 * np.sqrt(num_r), (np.sqrt(num_g), np.sqrt(num_r))
        assert not bad, f'weights further from the float64 rerun than twice the float32 oracle: {bad[:6]}'
