"""ctypes binding of the C ABI in ``include/aie4ml_b200.h``.

There is no CPU fallback: if the shared library has not been built, loading fails with an
error that says how to build it, and every operator call goes through the CUDA kernels.
"""

from __future__ import annotations

import ctypes
from ctypes import c_char_p, c_int, c_int64, c_void_p
from pathlib import Path
from typing import Optional

LIB_NAME = 'libaie4ml_b200.so'
LIB_PATH = Path(__file__).resolve().parent / LIB_NAME

A4C_OK = 0
A4C_ERR_INVALID_ARG = -1
A4C_ERR_ALIGNMENT = -2
A4C_ERR_UNSUPPORTED = -3
A4C_ERR_CUDA = -4
A4C_ERR_TOO_LARGE = -5
A4C_ERR_DEVICE_TIMEOUT = -6

ALGO_AUTO, ALGO_SIMT, ALGO_TCGEN05, ALGO_TCGEN05_PAIR = 0, 1, 2, 3
OPT_ROWOP_PATH = 0
OPT_BMM_PATH = 1
OPT_ROWOP_CHUNKS_PER_LANE = 2
OPT_ROWOP_MIN_STAGES = 3
OPT_ROWOP_CONTIG_COPY = 6
OPT_MLP_PATH = 4
OPT_DENSE_RESIDENT_W = 5
OPT_FLOAT_DENSE_PATH = 7
OPT_DENSE_PANEL_MIB = 8
OPT_WIDE_DENSE_PATH = 9
OPT_DENSE_LN_PATH = 10

# name -> (restype, argtypes); mirrors the header declaration by declaration
SIGNATURES = {
    'a4c_version': (c_int, []),
    'a4c_error_string': (c_char_p, [c_int]),
    'a4c_last_cuda_error': (c_char_p, []),
    'a4c_device_status': (c_int, [ctypes.POINTER(c_int), c_void_p]),
    'a4c_dense_i8': (c_int, [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_int64, c_int64, c_int, c_int,
                             c_int, c_int, c_int, c_int, c_int, c_int, c_void_p]),
    'a4c_bmm_i8': (c_int, [c_void_p, c_int64, c_int64, c_void_p, c_int64, c_int64, c_void_p, c_int64, c_int64, c_int64,
                           c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p]),
    'a4c_layernorm_i8': (c_int, [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_int64, c_int64,
                                 c_int, c_int, c_int, c_int, c_int, c_void_p]),
    'a4c_set_option': (c_int, [c_int, c_int]),
    'a4c_mlp_i8': (c_int, [c_void_p, c_int64, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                           c_int, c_void_p, c_int64, c_int, c_int64, c_void_p]),
    'a4c_mlp_i8_single_kernel': (c_int, [c_int, c_void_p, c_int, c_int64]),
    'a4c_mlp_i8_static': (c_int, [c_void_p, c_int64, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                  c_void_p, c_int, c_void_p, c_int64, c_int, c_int64, ctypes.POINTER(c_int), c_void_p]),
    'a4c_softmax_i8': (c_int, [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_int64, c_int, c_int, c_int,
                               c_int, c_int, c_int, c_int, c_int, c_int, c_void_p]),
    'a4c_dense_i16': (c_int, [c_void_p, c_int64, c_void_p, c_int, c_int64, c_void_p, c_void_p, c_int64, c_int64, c_int,
                              c_int, c_int, c_int, c_int, c_int, c_void_p]),
    'a4c_dense_ta': (c_int, [c_void_p, c_int, c_int64, c_int64, c_void_p, c_int, c_int64, c_void_p, c_void_p, c_int64,
                             c_int64, c_int64, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p]),
    'a4c_bmm_i16': (c_int, [c_void_p, c_int64, c_int64, c_void_p, c_int, c_int64, c_int64, c_void_p, c_int64, c_int64,
                            c_int64, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p]),
    'a4c_dense_f': (c_int, [c_void_p, c_int, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_int64, c_int64, c_int, c_int,
                            c_int, c_void_p]),
    'a4c_bmm_f': (c_int, [c_void_p, c_int, c_int64, c_int64, c_void_p, c_int64, c_int64, c_void_p, c_int64, c_int64, c_int64,
                          c_int, c_int, c_int, c_int, c_int, c_void_p]),
    'a4c_add_f': (c_int, [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_int64, c_int64, c_int, c_void_p]),
    'a4c_add_layernorm_i8': (c_int, [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int64,
                                     c_int64, c_int, c_int, c_int, c_int, c_int, c_void_p]),
    'a4c_dense_add_layernorm_supported': (c_int, [c_int64, c_int, c_int, c_int64, c_int64, c_int64, c_int64, c_int, c_int,
                                                  c_int, c_int, c_int]),
    'a4c_dense_add_layernorm_i8': (c_int, [c_void_p, c_int64, c_int, c_void_p, c_int64, c_void_p, c_int, c_int, c_void_p,
                                           c_int64, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int, c_int, c_int,
                                           c_int, c_int, c_int, c_void_p]),
    'a4c_attention_i8_supported': (c_int, [c_void_p, c_int64, c_int64, c_void_p, c_int64, c_int64, c_void_p, c_int64,
                                           c_int64, c_void_p, c_int64, c_int64, c_int64, c_int, c_int, c_int, c_int,
                                           c_int, c_int, c_int, c_int, c_int, c_int]),
    'a4c_attention_i8': (c_int, [c_void_p, c_int64, c_int64, c_void_p, c_int64, c_int64, c_void_p, c_int64, c_int64,
                                 c_void_p, c_int64, c_int64, c_int64, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                 c_int, c_int, c_int, c_int, c_int, c_int, c_void_p]),
    'a4c_attention_heads_i8_supported': (c_int, [c_void_p, c_int64, c_int64, c_int64, c_void_p, c_int64, c_int64, c_int64,
                                                 c_void_p, c_int64, c_int64, c_int64, c_void_p, c_int64, c_int64, c_int64,
                                                 c_int64, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                                 c_int, c_int]),
    'a4c_attention_heads_i8': (c_int, [c_void_p, c_int64, c_int64, c_int64, c_void_p, c_int64, c_int64, c_int64, c_void_p,
                                       c_int64, c_int64, c_int64, c_void_p, c_int64, c_int64, c_int64, c_int64, c_int, c_int,
                                       c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                       c_void_p]),
    'a4c_add_sat': (c_int, [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_int64, c_int64, c_int, c_int,
                            c_int, c_void_p]),
}


class A4cError(RuntimeError):
    def __init__(self, code: int, where: str, detail: str):
        super().__init__(f'{where}: {detail} (code {code})')
        self.code = code


_lib: Optional[ctypes.CDLL] = None


def load() -> ctypes.CDLL:
    """Load the library once; raises if it is missing (no fallback path exists)."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise RuntimeError(
            f'{LIB_PATH} is missing: the CUDA kernels have not been built. '
            'Run `python -m aie4ml_b200.build` (needs nvcc); there is no CPU fallback.')
    lib = ctypes.CDLL(str(LIB_PATH))
    for name, (restype, argtypes) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError here means the library is stale
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = lib
    return lib


def check(rc: int, where: str) -> None:
    if rc == A4C_OK:
        return
    lib = load()
    detail = lib.a4c_error_string(rc).decode()
    if rc == A4C_ERR_CUDA:
        detail += ': ' + lib.a4c_last_cuda_error().decode()
    raise A4cError(rc, where, detail)


def device_status(stream: int = 0) -> int:
    """Synchronise ``stream`` and return the device status word (0 = healthy).  Raises on a
    bounded-wait timeout reported by a kernel."""
    lib = load()
    status = c_int(0)
    rc = lib.a4c_device_status(ctypes.byref(status), c_void_p(stream))
    if rc == A4C_ERR_DEVICE_TIMEOUT:
        raise A4cError(rc, 'a4c_device_status', f'kernel wait {status.value} gave up')
    check(rc, 'a4c_device_status')
    return status.value
