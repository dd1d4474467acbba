"""Build libkvm_b200.so (sm_100a only) in-tree with nvcc.  `python -m kvm_b200.build [--force] [--verbose]`."""
from __future__ import annotations

import os
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / 'csrc'
LIB = PKG / 'libkvm_b200.so'
CLI = PKG / 'kvm_exec'
NVCC = os.environ.get('NVCC', '/usr/local/cuda/bin/nvcc')
CXX = os.environ.get('CXX', 'g++')
FLAGS = ['-gencode', 'arch=compute_100a,code=sm_100a', '-O3', '-std=c++17', '-lineinfo', '-shared', '-Xcompiler', '-fPIC',
         '--expt-relaxed-constexpr', '--extended-lambda', '-Xcudafe', '--diag_suppress=177']


def sources():
    return sorted(CSRC.glob('*')) + [PKG.parent / 'include' / 'kvm_b200.h', PKG.parent / 'include' / 'kvm_ops.def']


def stale() -> bool:
    if not LIB.exists():
        return True
    t = LIB.stat().st_mtime
    return any(s.stat().st_mtime > t for s in sources())


def build(force: bool = False, verbose: bool = False) -> Path:
    if not force and not stale():
        return LIB
    cmd = [NVCC, *FLAGS, *(['-Xptxas', '-v'] if verbose else []), str(CSRC / 'kvm_exec.cu'), '-o', str(LIB), '-lcudart']
    r = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or r.returncode:
        sys.stderr.write(r.stdout + r.stderr)
    if r.returncode:
        raise RuntimeError(f'nvcc failed ({r.returncode}): {" ".join(cmd)}')
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
