"""Builds ``libunit_b200.so`` in-tree with nvcc for sm_100a (no JIT cache)."""
from __future__ import annotations

import os
import shutil
import subprocess

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, 'libunit_b200.so')
_SOURCES = [os.path.join(_HERE, 'csrc', 'unit_abi.cu')]
_DEPS = _SOURCES + [os.path.join(_HERE, 'csrc', 'igemm_sm100.cuh'), os.path.join(_HERE, 'csrc', 'tensor_peak.cuh'),
                    os.path.join(os.path.dirname(_HERE), 'include', 'unit_b200.h')]


def _nvcc() -> str:
    for cand in (shutil.which('nvcc'), '/usr/local/cuda/bin/nvcc'):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError('nvcc not found: unit_b200 needs the CUDA toolkit to build its kernels')


def is_fresh() -> bool:
    if not os.path.exists(LIB_PATH):
        return False
    t = os.path.getmtime(LIB_PATH)
    return all(os.path.getmtime(s) <= t for s in _DEPS)


def build(force: bool = False, verbose: bool = False) -> str:
    if is_fresh() and not force:
        return LIB_PATH
    cmd = [_nvcc(), '-gencode', 'arch=compute_100a,code=sm_100a', '-lineinfo', '-O3', '-std=c++17',
           '-shared', '-Xcompiler', '-fPIC', '-o', LIB_PATH] + _SOURCES
    if verbose:
        cmd.insert(1, '-Xptxas')
        cmd.insert(2, '-v')
    subprocess.run(cmd, check=True)
    return LIB_PATH


if __name__ == '__main__':
    print(build(force=True, verbose=True))
