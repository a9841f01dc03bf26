import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
for p in (str(ROOT), str(ROOT / 'tests' / 'golden')):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line('markers', 'gpu: needs a CUDA device (run on the B200 box)')


def pytest_collection_modifyitems(config, items):
    try:
        import torch

        has_gpu = torch.cuda.is_available()
    except Exception:  # pragma: no cover
        has_gpu = False
    if has_gpu:
        return
    skip = pytest.mark.skip(reason='no CUDA device')
    for item in items:
        if 'gpu' in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope='session')
def oracle_c():
    """ctypes handle of the C edition of the oracle (built on demand)."""
    import ctypes
    import subprocess

    so = ROOT / 'oracle' / 'liboracle.so'
    src = ROOT / 'oracle' / 'oracle_c.c'
    if not so.exists() or so.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(['make', '-C', str(ROOT / 'oracle')], check=True, capture_output=True)
    return ctypes.CDLL(str(so))


@pytest.fixture(scope='session')
def oracle_c_native(tmp_path_factory):
    """The C oracle built for THIS host's CPU (-march=native), the build the benchmark times: on a CPU with
    AVX-512 VNNI its matrix products take the vpdpbusd path, which the portable build never compiles."""
    import ctypes
    import subprocess

    out = tmp_path_factory.mktemp('oracle_native') / 'liboracle_native.so'
    subprocess.run(['make', '-C', str(ROOT / 'oracle'), f'OUT={out}', 'ARCH=-march=native'], check=True,
                   capture_output=True)
    return ctypes.CDLL(str(out))
