"""Host handle of the B200 executor: ctypes over libkvm_b200.so (include/kvm_b200.h).

`Executor` mirrors the reference's `MvmExec` (mvm_exec.cu:492-1677): add_buffer -> submit -> start / finish -> read_buffer,
plus `load(bundle)`, which does what the reference CLI does with a bundle directory (mvm_exec.cu:2055-2076: create every
buffer of metadata.json with its init, then submit tasks / successors / args).  There is no CPU fallback: if the shared
library is missing or no sm_100 GPU is present, construction raises.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import numpy as np

from . import abi
from .bundle import Bundle, load_bundle

_LIB_PATH = Path(__file__).resolve().parent / 'libkvm_b200.so'
_lib = None

INIT_FILL, INIT_VALUES, INIT_SEEDED, INIT_NONE = 0, 1, 2, 3
CFG_NO_TENSOR_CORES = 1
CFG_PAIR_TILES = 2
CFG_CHAIN = 4
CFG_STATIC = 8
CFG_DYNAMIC = 16


class KvmError(RuntimeError):
    def __init__(self, code, text):
        super().__init__(f'[{code} {abi.err_name(code) if code > 0 else "host"}] {text}')
        self.code = code


class KvmConfig(C.Structure):
    _fields_ = [('device', C.c_int32), ('workers', C.c_int32), ('trace', C.c_int32), ('timeout_ms', C.c_int32), ('num_vars', C.c_int32),
                ('flags', C.c_int32)]


class KvmInit(C.Structure):
    _fields_ = [('kind', C.c_int32), ('draws', C.c_int32), ('fill', C.c_double), ('data', C.c_void_p), ('seed', C.c_uint64),
                ('bias', C.c_float), ('coef', C.c_float)]


class KvmResult(C.Structure):
    _fields_ = [('status', C.c_int32), ('done', C.c_int32), ('admitted', C.c_int32), ('err_task', C.c_int32), ('err_a', C.c_int32),
                ('err_b', C.c_int32), ('ms', C.c_float), ('busy_frac', C.c_float)]


# name -> (restype, argtypes): every symbol include/kvm_b200.h declares
SYMBOLS = {
    'kvm_create': (C.c_int, [C.POINTER(KvmConfig), C.POINTER(C.c_void_p)]),
    'kvm_destroy': (None, [C.c_void_p]),
    'kvm_add_buffer': (C.c_int, [C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.POINTER(KvmInit)]),
    'kvm_bind_buffer': (C.c_int, [C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_int32]),
    'kvm_buffer_ptr': (C.c_void_p, [C.c_void_p, C.c_int32]),
    'kvm_write_buffer': (C.c_int, [C.c_void_p, C.c_int32, C.c_void_p, C.c_size_t, C.c_size_t]),
    'kvm_read_buffer_raw': (C.c_int, [C.c_void_p, C.c_int32, C.c_void_p, C.c_size_t, C.c_size_t]),
    'kvm_read_buffer': (C.c_int, [C.c_void_p, C.c_int32, C.POINTER(C.c_float), C.c_size_t]),
    'kvm_set_version': (C.c_int, [C.c_void_p, C.c_int32, C.c_int32]),
    'kvm_get_version': (C.c_int, [C.c_void_p, C.c_int32, C.POINTER(C.c_int32)]),
    'kvm_submit': (C.c_int, [C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p, C.c_int32, C.c_void_p, C.c_int32]),
    'kvm_validate_batch': (C.c_int, [C.c_void_p, C.c_int32, C.c_void_p, C.c_int32, C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_char_p, C.c_size_t]),
    'kvm_submit_bundle_dir': (C.c_int, [C.c_void_p, C.c_char_p]),
    'kvm_load_bundle_dir': (C.c_int, [C.c_void_p, C.c_char_p]),
    'kvm_buffer_count': (C.c_int, [C.c_void_p]),
    'kvm_buffer_info': (C.c_int, [C.c_void_p, C.c_int32, C.POINTER(C.c_int32), C.POINTER(C.c_int32), C.POINTER(C.c_int32)]),
    'kvm_buffer_name': (C.c_char_p, [C.c_void_p, C.c_int32]),
    'kvm_buffer_index': (C.c_int, [C.c_void_p, C.c_char_p]),
    'kvm_variable_id': (C.c_int, [C.c_void_p, C.c_char_p]),
    'kvm_start': (C.c_int, [C.c_void_p]),
    'kvm_close': (C.c_int, [C.c_void_p]),
    'kvm_set_stream': (C.c_int, [C.c_void_p, C.c_void_p]),
    'kvm_finish': (C.c_int, [C.c_void_p, C.POINTER(KvmResult)]),
    'kvm_run': (C.c_int, [C.c_void_p, C.POINTER(KvmResult)]),
    'kvm_run_steps': (C.c_int, [C.c_void_p, C.c_int32, C.POINTER(KvmResult)]),
    'kvm_rearm': (C.c_int, [C.c_void_p]),
    'kvm_clear_tasks': (C.c_int, [C.c_void_p]),
    'kvm_task_counts': (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32]),
    'kvm_trace': (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32]),
    'kvm_trace_detail': (C.c_int, [C.c_void_p, C.c_void_p, C.c_int32]),
    'kvm_ipc_export': (C.c_int, [C.c_void_p, C.c_int32, C.c_void_p]),
    'kvm_ipc_open': (C.c_int, [C.c_void_p, C.c_void_p, C.POINTER(C.c_void_p)]),
    'kvm_ipc_close': (C.c_int, [C.c_void_p, C.c_void_p]),
    'kvm_launch_info': (C.c_int, [C.c_void_p, C.POINTER(C.c_int32), C.POINTER(C.c_int32), C.POINTER(C.c_int32)]),
    'kvm_plan_info': (C.c_int, [C.c_void_p, C.POINTER(C.c_int32), C.POINTER(C.c_int32), C.POINTER(C.c_float)]),
    'kvm_tc_task_count': (C.c_int, [C.c_void_p]),
    'kvm_last_error': (C.c_char_p, [C.c_void_p]),
    'kvm_read_f32_noalloc': (C.c_int, [C.c_int32, C.c_void_p, C.c_int32, C.c_size_t, C.POINTER(C.c_float), C.c_void_p]),
    'kvm_noalloc_last_error': (C.c_char_p, []),
    'kvm_err_name': (C.c_char_p, [C.c_int32]),
    'kvm_op_arity': (C.c_int, [C.c_int32]),
    'kvm_op_name': (C.c_char_p, [C.c_int32]),
}


def lib():
    """The loaded shared library with typed entry points. Raises if it has not been built (python -m kvm_b200.build)."""
    global _lib
    if _lib is None:
        if not _LIB_PATH.exists():
            raise KvmError(-6, f'{_LIB_PATH} not found: build it with `python -m kvm_b200.build` (there is no CPU fallback)')
        L = C.CDLL(str(_LIB_PATH))
        for name, (res, args) in SYMBOLS.items():
            f = getattr(L, name)
            f.restype, f.argtypes = res, args
        _lib = L
    return _lib


def validate_batch(tasks, succ, args, nbufs, nvars=64) -> str:
    """The C library's host check of one batch (no GPU needed): '' if well formed, else the first problem."""
    tasks = np.ascontiguousarray(tasks, dtype=abi.TASK_DTYPE)
    succ = np.ascontiguousarray(succ, dtype=np.int32)
    args = np.ascontiguousarray(args, dtype=np.int32)
    msg = C.create_string_buffer(512)
    lib().kvm_validate_batch(tasks.ctypes.data, len(tasks), succ.ctypes.data, len(succ), args.ctypes.data, len(args), nbufs, nvars, msg, 512)
    return msg.value.decode()


def bf16_bits(a: np.ndarray) -> np.ndarray:
    """float32 -> raw bf16 bits (round to nearest even)."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
    return ((u + np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1))) >> np.uint32(16)).astype(np.uint16)


class Executor:
    def __init__(self, device=0, workers=0, trace=False, timeout_ms=0, num_vars=0, flags=0):
        self._h = C.c_void_p()
        self.L = lib()
        cfg = KvmConfig(device, workers, int(trace), timeout_ms, num_vars, flags)
        r = self.L.kvm_create(C.byref(cfg), C.byref(self._h))
        if r != 0:
            raise KvmError(r, 'kvm_create failed (no sm_100 device or CUDA error; see stderr)')
        self.bundle: Bundle | None = None
        self.names: dict[str, int] = {}
        self.meta: list[dict] = []

    # ---- lifetime
    def close(self):
        if self._h:
            self.L.kvm_destroy(self._h)
            self._h = C.c_void_p()

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _check(self, r):
        if r != 0:
            raise KvmError(r, (self.L.kvm_last_error(self._h) or b'').decode())
        return r

    # ---- buffers
    def add_buffer(self, rows, cols, dtype=0, init=None, name=None) -> int:
        """init: None (zeros) | number (fill) | ndarray (values) | ('seeded', seed, draws, bias, coef) | 'none'."""
        ki = KvmInit()
        keep = None
        if init is None:
            ki.kind, ki.fill = INIT_FILL, 0.0
        elif isinstance(init, str) and init == 'none':
            ki.kind = INIT_NONE
        elif isinstance(init, (int, float)):
            ki.kind, ki.fill = INIT_FILL, float(init)
        elif isinstance(init, tuple) and init[0] == 'seeded':
            ki.kind, ki.seed, ki.draws, ki.bias, ki.coef = INIT_SEEDED, init[1], init[2], init[3], init[4]
        else:
            a = np.asarray(init)
            if dtype == abi.DTYPES['bf16']:
                keep = a.astype(np.uint16) if a.dtype == np.uint16 else bf16_bits(a)
            else:
                keep = np.ascontiguousarray(a, dtype=np.int32 if dtype == abi.DTYPES['i32'] else np.float32)
            assert keep.size == rows * cols, f'init has {keep.size} elements, buffer {rows}x{cols}'
            ki.kind, ki.data = INIT_VALUES, keep.ctypes.data
        idx = self.L.kvm_add_buffer(self._h, rows, cols, dtype, C.byref(ki))
        if idx < 0:
            self._check(idx)
        self.meta.append({'name': name or f'buf{idx}', 'rows': rows, 'cols': cols, 'dtype': dtype})
        if name:
            self.names[name] = idx
        return idx

    def bind_buffer(self, dev_ptr, rows, cols, dtype=0, ld=None, name=None) -> int:
        idx = self.L.kvm_bind_buffer(self._h, dev_ptr, rows, cols, ld or cols, dtype)
        if idx < 0:
            self._check(idx)
        self.meta.append({'name': name or f'buf{idx}', 'rows': rows, 'cols': cols, 'dtype': dtype})
        if name:
            self.names[name] = idx
        return idx

    def index(self, buf) -> int:
        return buf if isinstance(buf, int) else self.names[buf]

    def ipc_export(self, buf) -> bytes:
        """64-byte handle of a buffer this executor allocated, for an executor in another process of the node (kvm_ipc_export)."""
        h = C.create_string_buffer(64)
        self._check(self.L.kvm_ipc_export(self._h, self.index(buf), h))
        return h.raw

    def ipc_open(self, handle: bytes) -> int:
        """Device pointer of a peer's exported buffer mapped into this process (kvm_ipc_open)."""
        p = C.c_void_p()
        self._check(self.L.kvm_ipc_open(self._h, C.c_char_p(handle), C.byref(p)))
        return p.value

    def buffer_ptr(self, buf) -> int:
        return self.L.kvm_buffer_ptr(self._h, self.index(buf))

    def write_buffer(self, buf, a: np.ndarray, offset_elems=0):
        i = self.index(buf)
        dt = self.meta[i]['dtype']
        if dt == abi.DTYPES['bf16']:
            a = a if a.dtype == np.uint16 else bf16_bits(a)
        else:
            a = np.ascontiguousarray(a, dtype=np.int32 if dt == abi.DTYPES['i32'] else np.float32)
        self._check(self.L.kvm_write_buffer(self._h, i, a.ctypes.data, a.nbytes, offset_elems * abi.DTYPE_BYTES[dt]))
        self._keep = a

    def read_buffer(self, buf) -> np.ndarray:
        """Contents as a [rows, cols] array: float32 for f32 / bf16 storage (widened exactly), int32 for i32."""
        i = self.index(buf)
        m = self.meta[i]
        n = m['rows'] * m['cols']
        if m['dtype'] == abi.DTYPES['i32']:
            out = np.empty(n, np.int32)
            self._check(self.L.kvm_read_buffer_raw(self._h, i, out.ctypes.data, out.nbytes, 0))
        else:
            out = np.empty(n, np.float32)
            self._check(self.L.kvm_read_buffer(self._h, i, out.ctypes.data_as(C.POINTER(C.c_float)), n))
        return out.reshape(m['rows'], m['cols'])

    # ---- versions
    def set_version(self, var, v):
        self._check(self.L.kvm_set_version(self._h, var, v))

    def get_version(self, var) -> int:
        v = C.c_int32()
        self._check(self.L.kvm_get_version(self._h, var, C.byref(v)))
        return v.value

    # ---- tasks
    def submit(self, tasks: np.ndarray, succ: np.ndarray, args: np.ndarray):
        tasks = np.ascontiguousarray(tasks, dtype=abi.TASK_DTYPE)
        succ = np.ascontiguousarray(succ, dtype=np.int32)
        args = np.ascontiguousarray(args, dtype=np.int32)
        self._check(self.L.kvm_submit(self._h, tasks.ctypes.data, len(tasks), succ.ctypes.data, len(succ), args.ctypes.data, len(args)))

    def load(self, bundle) -> 'Executor':
        """Create the bundle's buffers (metadata.json order, with their inits), set base versions, submit its tasks."""
        b = bundle if isinstance(bundle, Bundle) else load_bundle(bundle)
        for spec in b.buffers:
            self.add_bundle_buffer(b, spec)
        for v in b.metadata.get('variables', []):
            if v.get('base_version', 0):
                self.set_version(v['id'], v['base_version'])
        self.submit(b.tasks, b.succ, b.args)
        self.bundle = b
        return self

    def load_dir(self, path) -> 'Executor':
        """The same through the C library's own loader (kvm_load_bundle_dir reads metadata.json itself): what a C++ host or the
        kvm_exec tool does with a bundle directory."""
        self._check(self.L.kvm_load_bundle_dir(self._h, str(path).encode()))
        rows, cols, dt = C.c_int32(), C.c_int32(), C.c_int32()
        for i in range(len(self.meta), self.L.kvm_buffer_count(self._h)):
            self._check(self.L.kvm_buffer_info(self._h, i, C.byref(rows), C.byref(cols), C.byref(dt)))
            name = self.L.kvm_buffer_name(self._h, i).decode() or f'buf{i}'
            self.meta.append({'name': name, 'rows': rows.value, 'cols': cols.value, 'dtype': dt.value})
            self.names[name] = i
        return self

    def add_bundle_buffer(self, b: Bundle, spec: dict) -> int:
        """One buffer of a bundle's metadata with its init (fill / values / seeded / file)."""
        init, dt = spec['init'], spec['dtype']
        kind = init['kind']
        if kind == 'fill':
            arg = init['value']
        elif kind == 'values':
            arg = np.array(init['values'], dtype=np.int32 if dt == 1 else np.float32)
        elif kind == 'seeded':
            arg = ('seeded', init['seed'], init['draws'], init['bias'], init['coef'])
        elif kind == 'file':
            raw = b.init_bytes(spec)
            arg = np.frombuffer(raw, dtype='<u2' if dt == 2 else '<i4' if dt == 1 else '<f4')
        else:
            raise KvmError(-3, f"buffer {spec['name']!r}: unknown init kind {kind!r}")
        return self.add_buffer(spec['rows'], spec['cols'], dt, arg, name=spec['name'])

    def rearm(self):
        self._check(self.L.kvm_rearm(self._h))

    def clear_tasks(self):
        self._check(self.L.kvm_clear_tasks(self._h))

    def start(self):
        self._check(self.L.kvm_start(self._h))

    def set_stream(self, cuda_stream: int):
        """Launch on the caller's stream (a cudaStream_t value, e.g. torch.cuda.current_stream().cuda_stream) from now on."""
        self._check(self.L.kvm_set_stream(self._h, C.c_void_p(cuda_stream)))

    def finish(self, check=True) -> KvmResult:
        res = KvmResult()
        r = self.L.kvm_finish(self._h, C.byref(res))
        if check and r != 0:
            raise KvmError(r, (self.L.kvm_last_error(self._h) or b'').decode())
        return res

    def run(self, check=True) -> KvmResult:
        res = KvmResult()
        r = self.L.kvm_run(self._h, C.byref(res))
        if check and r != 0:
            raise KvmError(r, (self.L.kvm_last_error(self._h) or b'').decode())
        return res

    def run_steps(self, steps, check=True) -> KvmResult:
        res = KvmResult()
        r = self.L.kvm_run_steps(self._h, steps, C.byref(res))
        if check and r != 0:
            raise KvmError(r, (self.L.kvm_last_error(self._h) or b'').decode())
        return res

    def task_counts(self, n=None):
        n = n if n is not None else len(self.bundle.tasks)
        ex, ob = np.empty(n, np.int32), np.empty(n, np.int32)
        self._check(self.L.kvm_task_counts(self._h, ex.ctypes.data, ob.ctypes.data, n))
        return ex, ob

    def trace(self, n=None):
        n = n if n is not None else len(self.bundle.tasks)
        s, e, sm = np.empty(n, np.uint64), np.empty(n, np.uint64), np.empty(n, np.int32)
        self._check(self.L.kvm_trace(self._h, s.ctypes.data, e.ctypes.data, sm.ctypes.data, n))
        return s, e, sm

    def trace_detail(self, n=None):
        """Per task the packed prologue / stage-wait times of a streamed GEMV on the static path (see kvm_trace_detail)."""
        n = n if n is not None else len(self.bundle.tasks)
        d = np.empty(n, np.int32)
        self._check(self.L.kvm_trace_detail(self._h, d.ctypes.data, n))
        return d

    def plan_info(self):
        """(runs on the static path?, with the stream ring?, planner's estimate of one run in us) of the prepared program."""
        a, b, us = C.c_int32(), C.c_int32(), C.c_float()
        self._check(self.L.kvm_plan_info(self._h, C.byref(a), C.byref(b), C.byref(us)))
        return bool(a.value), bool(b.value), us.value

    def tc_task_count(self) -> int:
        return self.L.kvm_tc_task_count(self._h)

    def launch_info(self):
        w, t, s = C.c_int32(), C.c_int32(), C.c_int32()
        self._check(self.L.kvm_launch_info(self._h, C.byref(w), C.byref(t), C.byref(s)))
        return w.value, t.value, s.value
