"""Build the CUDA kernels into spgt_b200/libspgt_b200.so for sm_100a with nvcc (no torch headers involved).

    python -m spgt_b200.build [--force]

The library is built in-tree so that it travels with the source tree; it is plain CUDA-runtime code behind a
C ABI (include/spgt_b200.h) and is loaded with ctypes by spgt_b200._lib.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, 'csrc')
INCLUDE = os.path.join(os.path.dirname(PKG), 'include')
LIB = os.path.join(PKG, 'libspgt_b200.so')
OBJ = os.path.join(PKG, 'build')
SOURCES = ['abi.cu', 'datamove.cu', 'attention.cu', 'attention_tc.cu', 'attention_bwd.cu', 'projection_bwd.cu', 'gemm.cu', 'tc_gemm.cu', 'tc_ffn.cu', 'scaler.cu', 'spectral.cu', 'metric.cu', 'darcy_solve.cu']
NVCC_FLAGS = ['-gencode', 'arch=compute_100a,code=sm_100a', '-lineinfo', '-O3', '-std=c++17',
              '-Xcompiler', '-fPIC', '-I', INCLUDE]


def _nvcc() -> str:
    for cand in (os.environ.get('NVCC'), shutil.which('nvcc'), '/usr/local/cuda/bin/nvcc'):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError('nvcc not found: cannot build libspgt_b200.so')


def _deps():
    files = [os.path.join(CSRC, f) for f in os.listdir(CSRC)] + [os.path.join(INCLUDE, 'spgt_b200.h')]
    return max(os.path.getmtime(f) for f in files)


def is_stale() -> bool:
    return not os.path.exists(LIB) or os.path.getmtime(LIB) < _deps()


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not is_stale():
        return LIB
    nvcc = _nvcc()
    os.makedirs(OBJ, exist_ok=True)

    def compile_one(src):
        obj = os.path.join(OBJ, src.replace('.cu', '.o'))
        cmd = [nvcc, *NVCC_FLAGS, '-c', os.path.join(CSRC, src), '-o', obj]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f'nvcc failed on {src}:\n{res.stdout}\n{res.stderr}')
        if verbose and res.stderr:
            print(res.stderr, file=sys.stderr)
        return obj

    with ThreadPoolExecutor(max_workers=len(SOURCES)) as ex:
        objs = list(ex.map(compile_one, SOURCES))
    res = subprocess.run([nvcc, '-shared', '-o', LIB, *objs, '-lcudart'], capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f'link failed:\n{res.stdout}\n{res.stderr}')
    return LIB


if __name__ == '__main__':
    print(build(force='--force' in sys.argv, verbose=True))
