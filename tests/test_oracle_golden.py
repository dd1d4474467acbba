"""The CPU oracle pinned to the reference: per-op fixtures produced by the reference's own pure-Python ops, the known-answer
vectors its tests hold (SplitMix64, seeded-buffer bit patterns, Philox, token sampling), and a two-step training run of the
reference compiler + CPU VM on this repo's gpt_micro workload (tests/golden/make_golden.py generated all three)."""
import hashlib
import json
from pathlib import Path

import numpy as np
import pytest

from kvm_b200 import abi
from kvm_b200.initgen import seeded_values, splitmix64
from oracle import ops_np
from oracle.ops_np import Buf

G = Path(__file__).resolve().parent / 'golden'
DT = {'f32': 0, 'i32': 1, 'bf16': 2}

_npz = np.load(G / 'ops_golden.npz')
_index = json.loads(bytes(_npz['index']).decode())

# Ops whose reference sums many terms in double before one float32 rounding: a vectorised double sum (pairwise) can land on the
# other side of a rounding boundary in the last bit. Everything else must match bit for bit.
ULP_OK = {'layernorm_fwd', 'rmsnorm_fwd', 'layernorm_bwd_dx', 'rmsnorm_bwd_dx', 'norm_bwd_params', 'attn_fwd', 'attn_bwd_delta', 'attn_bwd_dq', 'attn_bwd_dkv',
          'attn_decode', 'attn_decode_part', 'attn_decode_merge', 'gemv_bf16', 'softmax_ce_fwd', 'softmax_ce_bwd', 'softmax_ce_fused', 'softmax_ce_reduce',
          'gradnorm_partial', 'gradnorm_finish', 'gelu_fwd', 'gelu_bwd', 'act_fwd', 'act_bwd', 'silu_mul_fwd', 'matmul_tile', 'matmul_tile_bf16', 'rope_fwd', 'rope_bwd'}


@pytest.mark.parametrize('ci', range(len(_index)), ids=[f"{i}:{c['op']}" for i, c in enumerate(_index)])
def test_op_matches_reference(ci):
    case = _index[ci]
    op = case['op']
    bufs = {n: (None if dt is None else Buf(_npz[f'c{ci}.in.{n}'].copy(), DT[dt])) for n, dt in case['bufs'].items()}
    spec = abi.load_ops()[op]
    scal = {a.name: (float(np.float32(case['scalars'][a.name])) if a.type == 'f32' else int(case['scalars'][a.name])) for a in spec.args if a.type != 'buf'}
    ops_np.OPS[op](bufs, scal, exact_matmul=True)
    for n, b in bufs.items():
        if b is None:
            continue
        ref = _npz[f'c{ci}.out.{n}']
        if ref.dtype == np.int32:
            assert np.array_equal(b.a, ref), f'{op}.{n}'
            continue
        got = b.a.astype(np.float32)
        same = got.view(np.uint32) == ref.view(np.uint32)
        if same.all():
            continue
        assert op in ULP_OK, f'{op}.{n}: {int((~same).sum())} elements differ from the reference bit pattern'
        # at most one unit in the last place of the stored type
        ulp = np.spacing(np.abs(ref).astype(np.float32)) * (65536 if case['bufs'][n] == 'bf16' else 1)
        assert (np.abs(got.astype(np.float64) - ref.astype(np.float64)) <= 1.001 * ulp.astype(np.float64))[~same].all() and (~same).mean() < 0.05, f'{op}.{n}'


def test_splitmix64_known_answer():
    v = json.loads((G / 'vectors.json').read_text())
    assert [int(x) for x in splitmix64(0, np.arange(3))] == v['splitmix64_seed0'] == [0xE220A8397B1DCDAF, 0x6E789E6AA1B965F4, 0x06C45D188009454F]


def test_seeded_buffers_bit_patterns():
    v = json.loads((G / 'vectors.json').read_text())
    assert len(v['initgen']) >= 20
    for case in v['initgen']:
        bias = float(np.array([int(case['bias_bits'], 16)], np.uint32).view(np.float32)[0])
        coef = float(np.array([int(case['coef_bits'], 16)], np.uint32).view(np.float32)[0])
        got = seeded_values(case['seed'], case['n'], case['draws'], bias, coef).view(np.uint32)
        want = np.array([int(x, 16) for x in case['bits']], np.uint32)
        assert np.array_equal(got, want), case['seed']


def test_philox_and_sampling_vectors():
    v = json.loads((G / 'vectors.json').read_text())
    num = lambda xs: [int(x, 16) if isinstance(x, str) else int(x) for x in xs]
    for k in v['philox_kat']:
        assert ops_np.philox4x32_10(num(k['counter']), num(k['key'])) == num(k['out'])
    assert ops_np.philox4x32_10([0xFFFFFFFF] * 4, [0xFFFFFFFF] * 2) == [0x408F276D, 0x41C83B0E, 0xA20BC7C6, 0x6D5451FD]
    for c in v['sample_cases']:
        V, R = c['V'], c['rows']
        b = {'logits': Buf(np.array(c['logits'], np.float32).reshape(R, V), 0), 'out': Buf(np.zeros((R, 1), np.int32), 1), 'ctr': Buf(np.array([[c['ctr']]], np.int32), 1)}
        ops_np.sample(b, {'r0': 0, 'r1': R, 'V': V, 'temp': float(np.float32(c['temp'])), 'topk': c['topk'], 'seed': c['seed']})
        assert b['out'].a.reshape(-1).tolist() == c['expected'], (c['temp'], c['topk'])


def test_gpt_micro_against_reference_compiler_and_vm():
    from kvm_b200.workloads.gpt import build_training, preset
    from oracle.vm_np import VM
    gold = json.loads((G / 'gpt_micro_golden.json').read_text())
    b = build_training(preset('gpt_micro'), 2).to_bundle()
    # this repo's compiler packs the same bytes the reference compiler does from the same workload JSON
    assert hashlib.sha256(b.tasks.tobytes()).hexdigest() == gold['bundle_sha256']['tasks.bin']
    assert hashlib.sha256(b.succ.astype('<i4').tobytes()).hexdigest() == gold['bundle_sha256']['successors.bin']
    assert hashlib.sha256(b.args.astype('<i4').tobytes()).hexdigest() == gold['bundle_sha256']['args.bin']
    vm = VM(b).run()
    assert {b.metadata['variables'][k]['name']: v for k, v in vm.versions.items()} == gold['versions']
    for name, vals in gold['buffers'].items():
        got = vm.buffer(name).a.reshape(-1)
        np.testing.assert_allclose(got, np.array(vals, got.dtype), rtol=2e-7, atol=1e-12, err_msg=name)
    exact = sum(hashlib.sha256(buf.a.tobytes()).hexdigest() == gold['buffer_sha256'][spec['name']] for spec, buf in zip(b.buffers, vm.bufs))
    assert exact >= 0.9 * len(b.buffers), f'only {exact} of {len(b.buffers)} buffers are bit-identical to the reference VM'


@pytest.mark.parametrize('name', ['ref_gpt_tiny_f32', 'ref_gpt_tiny_bf16s'])
def test_reference_frontend_bundle_on_the_oracle(name):
    """A bundle directory written by the reference's own frontend + compiler (its gpt_tiny: RoPE, biases, untied head), run by the
    oracle VM, against the final state of the reference CPU VM (golden.npz): every buffer to float32 rounding."""
    from kvm_b200.bundle import load_bundle
    from oracle.vm_np import VM
    d = G / name
    z = np.load(d / 'golden.npz')
    meta = json.loads(bytes(z['meta']).decode())
    b = load_bundle(d)
    vm = VM(b).run()
    assert {b.metadata['variables'][k]['name']: v for k, v in vm.versions.items()} == meta['versions']
    worst = 0.0
    for k in z.files:
        if not k.startswith('buf.'):
            continue
        ref, got = z[k], vm.buffer(k[4:]).a.reshape(-1)
        if ref.dtype == np.int32:
            assert np.array_equal(got, ref), k
            continue
        den = float(np.sqrt((ref.astype(np.float64) ** 2).sum()))
        err = float(np.sqrt(((got.astype(np.float64) - ref) ** 2).sum())) / max(den, 1e-30)
        if 'attn.k.b' not in k:          # an exactly-zero gradient: what is computed is rounding noise (see tests/parity.py)
            worst = max(worst, err)
    assert worst <= (2e-6 if name.endswith('f32') else 4e-3), worst
