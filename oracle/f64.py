"""All-double rerun of the CPU oracle.  TEST INFRASTRUCTURE, not product code.

The acceptance criterion for float32 training asks that the weights stay "within 2x the reference's deviation from an f64
rerun": the reference has such a rerun in its float64 interpreter (`frontend/mvmfe/refvm.py`: the same program, every value a
Python float, no float32 rounding anywhere).  This module gives the oracle the same mode without a second copy of the ops:
it loads `oracle/ops_np.py` a second time with every `np.float32` replaced by `np.float64`, so each op follows the same
formulae and the same order of operations, only without the per-operation rounding to float32 (and without the rounding to
bf16 / tf32 storage, which the double rerun leaves out as well).  Buffers of a VM that uses it are float64 arrays.
"""
from __future__ import annotations

import types
from pathlib import Path

import numpy as np

_mod = None


def ops_f64():
    """The double-precision twin of oracle.ops_np (module object with the same OPS table)."""
    global _mod
    if _mod is None:
        src = (Path(__file__).resolve().parent / 'ops_np.py').read_text().replace('np.float32', 'np.float64')
        m = types.ModuleType('oracle.ops_np_f64')
        m.__file__ = str(Path(__file__).resolve().parent / 'ops_np.py')
        exec(compile(src, m.__file__ + ' (float64)', 'exec'), m.__dict__)
        keep = lambda x: np.asarray(x, dtype=np.float64)
        m.bf16_round = keep          # storage rounding does not exist in the double rerun
        m.tf32_round = keep
        _mod = m
    return _mod
