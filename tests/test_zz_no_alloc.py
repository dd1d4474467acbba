"""The allocation-free read-back (kvm_read_f32_noalloc) against the ordinary one (kvm_read_buffer), through the C ABI.

The ordinary entry point widens bf16 / i32 storage in a temporary it cudaMallocs; the allocation-free one uses a fixed scratch
array inside the library, for callers that must not allocate: a decode loop that reads tokens or logits back every step while
other streams (or a persistent executor) keep the GPU busy, where cudaMalloc / cudaFree would synchronise the whole device.
Two calls in a row share that array, so the second one is smaller and holds different data: stale contents of the first call
would show.  This file sorts last on purpose, so a failure here cannot hide another test's result.
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _noalloc(ex, buf, n):
    m = ex.meta[ex.index(buf)]
    out = np.full(n, np.nan, np.float32)
    r = ex.L.kvm_read_f32_noalloc(0, ex.buffer_ptr(buf), m['dtype'], n, out.ctypes.data_as(C.POINTER(C.c_float)), None)
    assert r == 0, ex.L.kvm_noalloc_last_error().decode()
    return out


def test_noalloc_read_matches_read_buffer_twice(kvm_lib):
    from kvm_b200.executor import Executor
    rng = np.random.default_rng(5)
    with Executor() as ex:
        a = rng.standard_normal((300, 1000)).astype(np.float32)
        b = rng.integers(-1000, 1000, (7, 333)).astype(np.int32)
        c = rng.standard_normal((5, 64)).astype(np.float32)
        ex.add_buffer(300, 1000, 2, a, name='a')      # bf16 storage
        ex.add_buffer(7, 333, 1, b, name='b')         # i32
        ex.add_buffer(5, 64, 0, c, name='c')          # f32
        first = _noalloc(ex, 'a', 300000)
        second = _noalloc(ex, 'b', 7 * 333)           # right after, smaller, other data: the scratch still holds `a`
        third = _noalloc(ex, 'c', 320)
        assert np.array_equal(first, ex.read_buffer('a').reshape(-1))      # exact: widening bf16 / int32 to float32 loses nothing
        assert np.array_equal(second, ex.read_buffer('b').reshape(-1).astype(np.float32))
        assert np.array_equal(third, ex.read_buffer('c').reshape(-1))
        # and against what was uploaded: bf16 storage holds the uploaded values rounded to nearest even
        from kvm_b200.executor import bf16_bits
        assert np.array_equal(first, (bf16_bits(a).astype(np.uint32) << 16).view(np.float32).reshape(-1))
        assert np.array_equal(second, b.reshape(-1).astype(np.float32)) and np.array_equal(third, c.reshape(-1))
        assert ex.L.kvm_noalloc_last_error() == b''          # a successful call leaves no stale message
        # exactly the maximum, on a stream of the caller's own (not the default stream)
        import torch
        big_src = rng.standard_normal((1024, 1024)).astype(np.float32)
        ex.add_buffer(1024, 1024, 2, big_src, name='big')
        stream = torch.cuda.Stream()
        out = np.full(1 << 20, np.nan, np.float32)
        r = ex.L.kvm_read_f32_noalloc(0, ex.buffer_ptr('big'), 2, 1 << 20, out.ctypes.data_as(C.POINTER(C.c_float)), C.c_void_p(stream.cuda_stream))
        assert r == 0, ex.L.kvm_noalloc_last_error().decode()
        assert np.array_equal(out, ex.read_buffer('big').reshape(-1))
        assert torch.cuda.current_device() == 0                  # the caller's current device is as it was
        # beyond the fixed scratch: refused with a message, nothing copied
        big = np.zeros(4, np.float32)
        r = ex.L.kvm_read_f32_noalloc(0, ex.buffer_ptr('a'), 2, (1 << 20) + 1, big.ctypes.data_as(C.POINTER(C.c_float)), None)
        assert r == -1 and b'exceed' in ex.L.kvm_noalloc_last_error()
