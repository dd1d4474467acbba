"""Task ABI v2 as seen from Python: the 64-byte task descriptor, buffer dtypes, error codes and the operator registry.

The descriptor layout follows the reference's `include/mvm_task_abi.h:11-29` (sixteen little-endian int32 fields) and the
registry is parsed from `include/kvm_ops.def`, the same text the CUDA dispatcher expands, so ids and arities cannot drift
between the host compiler, the CPU oracle and the device (the reference does the same in `runtime/abi.py:55-116`).
"""
from __future__ import annotations

import re
from dataclasses import dataclass
from functools import lru_cache
from pathlib import Path

import numpy as np

ABI_VERSION = 2
NO_VAR = -1
ABSENT_BUF = -1
MAX_ARGS = 20          # reference: MVM_MAX_ARGS, include/mvm_exec.cuh:58
NUM_PRIORITIES = 32    # reference: MVM_NBUCKETS, include/mvm_exec.cuh:51

TASK_FIELDS = ('op_id', 'succ_off', 'succ_cnt', 'indegree', 'priority', 'deadline_us', 'args_off', 'args_words',
               'wait_var', 'wait_ver', 'pub_var', 'pub_ver', 'workload_id', 'flags', 'reserved0', 'reserved1')
TASK_DTYPE = np.dtype([(f, '<i4') for f in TASK_FIELDS])
assert TASK_DTYPE.itemsize == 64

DTYPES = {'f32': 0, 'i32': 1, 'bf16': 2}
DTYPE_NAMES = {v: k for k, v in DTYPES.items()}
DTYPE_BYTES = {0: 4, 1: 4, 2: 2}

# Executor error codes (reference: MVM_ERRORS, include/mvm_exec.cuh:147-164) and op-pack codes (mvm_ops_gpt.cuh:181-194).
ERRORS = ('OK', 'BAD_OP', 'BAD_ARITY', 'BAD_BUF_INDEX', 'BAD_BUF', 'BOUNDS', 'BAD_VAR', 'VERSION_GAP', 'WAIT_VIOLATION',
          'DOUBLE_EXEC', 'BAD_RECORD', 'BAD_TASK', 'SLOTS', 'POOL', 'BATCH_TOO_LARGE', 'TIMEOUT', 'QUEUE_OVERFLOW',
          'BAD_CONFIG', 'PARK_STALL', 'TASK_LIMIT', 'ALIAS_RECORD')
OP_ERR_BASE = 1000
OP_ERRORS = {1: 'E_BUF', 2: 'E_DTYPE', 3: 'E_RANGE', 4: 'E_SHAPE', 5: 'E_TOKEN', 6: 'E_KVLEN', 7: 'E_SMEM'}

OPS_DEF = Path(__file__).resolve().parents[1] / 'include' / 'kvm_ops.def'


def err_name(code: int) -> str:
    if 0 <= code < len(ERRORS):
        return ERRORS[code]
    if code - OP_ERR_BASE in OP_ERRORS:
        return OP_ERRORS[code - OP_ERR_BASE]
    return f'UNKNOWN({code})'


@dataclass(frozen=True)
class OpArg:
    name: str
    type: str          # 'buf' | 'i32' | 'f32'
    optional: bool = False


@dataclass(frozen=True)
class OpSpec:
    name: str
    id: int
    args: tuple

    @property
    def arity(self) -> int:
        return len(self.args)


class AbiError(RuntimeError):
    pass


@lru_cache(maxsize=None)
def load_ops(path: Path = OPS_DEF) -> dict:
    """{name: OpSpec} in file order."""
    ops, ids = {}, {}
    line_re = re.compile(r'^KVM_OP\(\s*(\w+)\s*,\s*(\d+)\s*,\s*"([^"]*)"\s*\)')
    for ln, line in enumerate(Path(path).read_text().splitlines(), 1):
        if not line.startswith('KVM_OP('):
            continue
        m = line_re.match(line)
        if not m:
            raise AbiError(f'{path}:{ln}: unparsable operator line')
        name, op_id, sig = m.group(1), int(m.group(2)), m.group(3)
        args = []
        for item in filter(None, (s.strip() for s in sig.split(','))):
            an, _, at = item.partition(':')
            opt = at == 'buf?'
            at = 'buf' if opt else at
            if at not in ('buf', 'i32', 'f32'):
                raise AbiError(f'{path}:{ln}: bad argument {item!r}')
            args.append(OpArg(an, at, opt))
        if name in ops or op_id in ids or len(args) > MAX_ARGS:
            raise AbiError(f'{path}:{ln}: duplicate name/id or too many arguments: {name}')
        ops[name] = OpSpec(name, op_id, tuple(args))
        ids[op_id] = name
    return ops


@lru_cache(maxsize=None)
def ops_by_id() -> dict:
    return {o.id: o for o in load_ops().values()}


def f32_word(x: float) -> int:
    """float -> the int32 argument word holding its float32 bits."""
    return int(np.array([x], dtype='<f4').view('<i4')[0])


def word_f32(w: int) -> float:
    return float(np.array([w], dtype='<i4').view('<f4')[0])
