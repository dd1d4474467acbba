"""Build libkvm_b200.so (sm_100a only) in-tree with nvcc.  `python -m kvm_b200.build [--force] [--verbose]`."""
from __future__ import annotations

import os
import time
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / 'csrc'
LIB = PKG / 'libkvm_b200.so'
CLI = PKG / 'kvm_exec'
NVCC = os.environ.get('NVCC', '/usr/local/cuda/bin/nvcc')
CXX = os.environ.get('CXX', 'g++')
UNITS = ('kvm_exec', 'kvm_static')
FLAGS = ['-gencode', 'arch=compute_100a,code=sm_100a', '-O3', '-std=c++17', '-lineinfo', '-Xcompiler', '-fPIC',
         '--expt-relaxed-constexpr', '--extended-lambda', '-Xcudafe', '--diag_suppress=177']


# files that only one of the two translation units reads (everything else under csrc/ and include/ feeds both)
ONLY = {'kvm_exec': {'kvm_exec.cu', 'kvm_sched.cuh', 'kvm_host.inl', 'kvm_gemm_host.inl', 'kvm_static_host.inl', 'kvm_json.hpp'},
        'kvm_static': {'kvm_static.cu', 'kvm_static.cuh'}}


def sources(unit=None):
    skip = {'kvm_cli.cpp'} | (set().union(*(v for k, v in ONLY.items() if k != unit)) if unit else set())
    return [p for p in sorted(CSRC.glob('*')) if p.name not in skip] + [PKG.parent / 'include' / 'kvm_b200.h', PKG.parent / 'include' / 'kvm_ops.def']


def unit_stale(unit) -> bool:
    obj = PKG / f'_{unit}.o'
    return not obj.exists() or any(s.stat().st_mtime > obj.stat().st_mtime for s in sources(unit))


def stale() -> bool:
    if not LIB.exists():
        return True
    return any(unit_stale(u) for u in UNITS) or any((PKG / f'_{u}.o').stat().st_mtime > LIB.stat().st_mtime for u in UNITS)


def build(force: bool = False, verbose: bool = False) -> Path:
    """Two translation units (the ready-queue kernel + host code, the static-schedule kernel), compiled side by side, then linked."""
    if not force and not stale():
        return LIB
    objs, procs = [], []
    started = time.time()          # an object counts as built when its compile STARTED: a source edited while nvcc runs stays newer
    for unit in UNITS:
        obj = PKG / f'_{unit}.o'
        objs.append(obj)
        if not force and not unit_stale(unit):
            continue
        cmd = [NVCC, *FLAGS, *(['-Xptxas', '-v'] if verbose else []), '-c', str(CSRC / f'{unit}.cu'), '-o', str(obj)]
        procs.append((cmd, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)))
    for cmd, p in procs:
        out, err = p.communicate()
        if verbose or p.returncode:
            sys.stderr.write(out + err)
        if p.returncode:
            raise RuntimeError(f'nvcc failed ({p.returncode}): {" ".join(cmd)}')
        os.utime(cmd[-1], (started, started))
    cmd = [NVCC, '-gencode', 'arch=compute_100a,code=sm_100a', '-shared', *map(str, objs), '-o', str(LIB), '-lcudart']
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode:
        sys.stderr.write(r.stdout + r.stderr)
        raise RuntimeError(f'link failed ({r.returncode}): {" ".join(cmd)}')
    return LIB


def build_cli(force: bool = False) -> Path:
    """kvm_exec: the command-line runner (host C++ over the C ABI, no CUDA code of its own), next to the library."""
    src = CSRC / 'kvm_cli.cpp'
    if not force and CLI.exists() and CLI.stat().st_mtime >= max(src.stat().st_mtime, LIB.stat().st_mtime if LIB.exists() else 0):
        return CLI
    build(force)
    cmd = [CXX, '-O2', '-std=c++17', str(src), '-o', str(CLI), f'-L{PKG}', '-lkvm_b200', '-Wl,-rpath,$ORIGIN']
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode:
        sys.stderr.write(r.stdout + r.stderr)
        raise RuntimeError(f'g++ failed ({r.returncode}): {" ".join(cmd)}')
    return CLI


if __name__ == '__main__':
    print(build(force='--force' in sys.argv, verbose='--verbose' in sys.argv))
    print(build_cli(force='--force' in sys.argv))
