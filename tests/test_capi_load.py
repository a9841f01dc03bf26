"""The C-ABI library loads without a GPU and exports every symbol the public header declares."""

import ctypes
import re
from pathlib import Path

from aie4ml_b200 import lib as a4c

ROOT = Path(__file__).resolve().parent.parent
HEADER = (ROOT / 'include' / 'aie4ml_b200.h').read_text()


def declared_symbols():
    return re.findall(r'A4C_API\s+[\w\s\*]+?\b(a4c_\w+)\s*\(', HEADER)


def test_library_exports_every_declared_symbol():
    names = declared_symbols()
    assert len(names) >= 9 and len(set(names)) == len(names)
    handle = ctypes.CDLL(str(a4c.LIB_PATH))
    for name in names:
        assert hasattr(handle, name), f'{name} is declared in the header but not exported'


def test_binding_table_matches_header():
    assert set(a4c.SIGNATURES) == set(declared_symbols())
    lib = a4c.load()
    assert lib.a4c_version() >= 100
    assert lib.a4c_error_string(a4c.A4C_ERR_ALIGNMENT).decode().startswith('pointer or pitch')
    assert lib.a4c_error_string(12345).decode() == 'unknown error code'


def test_header_error_codes_match_binding():
    for name in ('A4C_ERR_INVALID_ARG', 'A4C_ERR_ALIGNMENT', 'A4C_ERR_UNSUPPORTED', 'A4C_ERR_CUDA', 'A4C_ERR_TOO_LARGE',
                 'A4C_ERR_DEVICE_TIMEOUT'):
        value = int(re.search(rf'#define {name} \((-?\d+)\)', HEADER).group(1))
        assert getattr(a4c, name) == value


def test_every_header_entry_cites_the_reference_or_says_it_has_none():
    # each kernel entry point's comment names the reference kernel file it replaces
    for kernel_file in ('dense_bias_relu.cpp', 'matmul.cpp', 'layer_norm.cpp', 'softmax.cpp', 'elementwise_add.cpp'):
        assert kernel_file in HEADER
