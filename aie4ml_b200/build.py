"""Builds the CUDA library in-tree: ``aie4ml_b200/libaie4ml_b200.so`` (sm_100a only).

``python -m aie4ml_b200.build`` (or ``build_library()``) compiles every ``csrc/*.cu`` with nvcc and
links one shared object that exports the C ABI of ``include/aie4ml_b200.h``.  Object files are
cached by source timestamp so an unchanged file is not recompiled.
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / 'csrc'
BUILD_DIR = PKG_DIR / 'csrc' / 'build'
LIB_PATH = PKG_DIR / 'libaie4ml_b200.so'

NVCC_FLAGS = [
    '-gencode', 'arch=compute_100a,code=sm_100a', '-lineinfo', '-O3', '-std=c++17',
    '-Xcompiler', '-fPIC', '-Xcompiler', '-fvisibility=hidden', '--expt-relaxed-constexpr',
]


def _nvcc() -> str:
    for cand in (os.environ.get('NVCC'), shutil.which('nvcc'), '/usr/local/cuda/bin/nvcc'):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError('nvcc not found; the CUDA library cannot be built')


def _stale(target: Path, deps) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(Path(d).stat().st_mtime > t for d in deps)


def build_library(verbose: bool = False, ptxas_info: bool = False) -> Path:
    nvcc = _nvcc()
    BUILD_DIR.mkdir(parents=True, exist_ok=True)
    headers = sorted(CSRC.glob('*.cuh')) + sorted(CSRC.glob('*.h')) + [PKG_DIR.parent / 'include' / 'aie4ml_b200.h']
    objects, jobs = [], []
    for src in sorted(CSRC.glob('*.cu')):
        obj = BUILD_DIR / (src.stem + '.o')
        objects.append(obj)
        if _stale(obj, [src, *headers]):
            cmd = [nvcc, *NVCC_FLAGS, '-ccbin', '/usr/bin/g++', '-c', str(src), '-o', str(obj)]
            if ptxas_info:
                cmd[1:1] = ['-Xptxas', '-v']
            jobs.append(cmd)

    def compile_one(cmd):
        if verbose:
            print(' '.join(cmd), flush=True)
        subprocess.run(cmd, check=True)

    # the translation units are independent: compile the stale ones side by side
    with ThreadPoolExecutor(max_workers=max(1, min(len(jobs), os.cpu_count() or 1))) as pool:
        list(pool.map(compile_one, jobs))
    if _stale(LIB_PATH, objects):
        cmd = [nvcc, '-shared', '-gencode', 'arch=compute_100a,code=sm_100a', '-ccbin', '/usr/bin/g++',
               '--cudart', 'static', '-o', str(LIB_PATH), *map(str, objects)]
        if verbose:
            print(' '.join(cmd), flush=True)
        subprocess.run(cmd, check=True)
    return LIB_PATH


if __name__ == '__main__':
    path = build_library(verbose=True, ptxas_info='--ptxas' in sys.argv)
    print(path)
