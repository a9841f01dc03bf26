"""Checker built on the CPU oracle: evaluates an exported lowered plan on a sample of the batch.

TEST INFRASTRUCTURE.  Used by the tests, by ``__graft_entry__.smoke()`` and by ``bench.py`` (its parity
field, its CPU-baseline leg and its ``--impl reference`` arm); the shipped package never imports it.

Every operator of a lowered graph is independent along the flattened leading axis (rows of a Dense or
row op, whole sequences of an encoder block), so the oracle's result for any subset of leading
indices equals the corresponding slice of its result for the whole batch.  That is what makes parity
at full benchmark sizes affordable: the device computes the whole batch, the oracle a few hundred
sampled units, and the two are compared bit for bit on those.

Two evaluators: ``oracle.run_plan`` (NumPy, the primary restatement) for small samples, and
``run_plan_c`` (the C edition, itself tested against the NumPy one) where a NumPy int64 matrix
product would take minutes (K = N = 8192).
"""

from __future__ import annotations

import ctypes
import os
import subprocess
import time
from pathlib import Path
from typing import Dict, Optional, Sequence, Tuple

import numpy as np

from . import c_api as C
from . import oracle

HERE = Path(__file__).resolve().parent


def load_c(native: bool = True, threads: Optional[int] = None):
    """Build (if needed) and load the C oracle.  ``native``: compile for this host's CPU into a temporary file
    (falls back to the portable in-tree build).  Returns (lib, description)."""
    lib = arch = None
    if native:
        out = Path('/tmp') / f'liboracle_native_{os.getpid()}.so'
        try:
            subprocess.run(['make', '-C', str(HERE), f'OUT={out}', 'ARCH=-march=native'], check=True,
                           capture_output=True, timeout=180)
            lib, arch = ctypes.CDLL(str(out)), 'native'
        except Exception:
            lib = None
    if lib is None:
        so = HERE / 'liboracle.so'
        if not so.exists() or so.stat().st_mtime < (HERE / 'oracle_c.c').stat().st_mtime:
            subprocess.run(['make', '-C', str(HERE)], check=True, capture_output=True)
        lib, arch = ctypes.CDLL(str(so)), 'x86-64-v3'
    lib.orc_num_threads.restype = ctypes.c_int
    lib.orc_gemm_path.restype = ctypes.c_int
    # all host threads, whatever the launcher exported (torchrun sets OMP_NUM_THREADS=1)
    n = threads or (len(os.sched_getaffinity(0)) if hasattr(os, 'sched_getaffinity') else os.cpu_count())
    lib.orc_set_threads(ctypes.c_int(int(n)))
    return lib, f"{arch}, {'AVX-512 VNNI' if lib.orc_gemm_path() else 'portable'} matrix products"


def run_plan_c(lib, plan: dict, inputs: Dict[str, np.ndarray]) -> Tuple[Dict[str, np.ndarray], float]:
    """Evaluate an exported plan with the C oracle.  Returns (graph outputs, seconds spent inside oracle calls:
    view ops and argument marshalling are not counted)."""
    env = {k: np.ascontiguousarray(v) for k, v in inputs.items()}
    params = plan['params']
    elapsed = 0.0
    for op in plan['ops']:
        kind = op['kind']
        if kind == 'slice':
            src = env[op['source']]
            for item in op['slices']:
                idx = [slice(None)] * src.ndim
                idx[op['axis']] = slice(item['start'], item['start'] + item['extent'])
                env[item['output']] = np.ascontiguousarray(src[tuple(idx)])
            continue
        if kind == 'concat':
            env[op['out']] = np.concatenate([env[n] for n in op['inputs']], axis=op['axis'])
            continue
        t0 = time.perf_counter()
        if kind == 'dense':
            if op.get('transpose_lhs') or op.get('acc_bits', 32) != 32 or op.get('lhs_dtype', 'int8') == 'int16':
                raise NotImplementedError(f"{op['name']}: the C oracle has no 16-bit or transposed-input Dense")
            a = env[op['lhs']]
            y = C.dense(lib, a.reshape(-1, a.shape[-1]), params[op['weight']], params[op['bias']] if op['bias'] else None,
                        shift=op['shift'], tok=op['rounding'], relu=op['relu'], out_dtype=op['out_dtype'])
            env[op['out']] = y.reshape(*a.shape[:-1], -1)
        elif kind == 'matmul':
            a, b = env[op['lhs']], env[op['rhs']]
            env[op['out']] = C.bmm(lib, a, b, shift=op['shift'], tok=op['rounding'], trans_a=op['transpose_lhs'],
                                   trans_b=op['transpose_rhs'], out_dtype=op['out_dtype'])
        elif kind == 'add':
            a = env[op['lhs']]
            env[op['out']] = C.add(lib, a.reshape(-1, a.shape[-1]), env[op['rhs']].reshape(-1, a.shape[-1]),
                                   shift=op['shift'], tok=op['rounding'], dtype=op['out_dtype']).reshape(a.shape)
        elif kind == 'layer_norm':
            a = env[op['lhs']]
            env[op['out']] = C.layer_norm(lib, a.reshape(-1, a.shape[-1]), params[op['gamma']], params[op['beta']],
                                          eps_q0=op['eps_q0'], out_shift=op['out_shift'], tok=op['rounding']).reshape(a.shape)
        elif kind == 'softmax':
            a = env[op['lhs']]
            env[op['out']] = C.softmax(lib, a.reshape(-1, a.shape[-1]), mode=op['approximation'], B=op['B'], S=op['S'],
                                       Dmax=op['Dmax'], inv_shift=op['inv_shift'], use_clb=op['use_clb'],
                                       exp_kq=op['exp_kq'], out_dtype=op['out_dtype']).reshape(a.shape)
        else:
            raise NotImplementedError(f'the C oracle has no {kind!r} op')
        elapsed += time.perf_counter() - t0
    return {name: env[name] for name in plan['outputs']}, elapsed


def sample_units(total: int, want: int, tile: int = 128, seed: int = 0) -> np.ndarray:
    """Sorted unique leading indices to check: the whole first and last `tile`-aligned groups' edges (first and last
    unit of the batch, both sides of the first and last tile boundary), one unit per evenly spaced tile across the
    middle, and seeded random ones, `want` in all (or every unit when the batch is smaller)."""
    total, want = int(total), int(want)
    if total <= want:
        return np.arange(total, dtype=np.int64)
    rng = np.random.default_rng(seed)
    picks = {0, 1, tile - 1, tile, total - tile - 1, total - tile, total - 2, total - 1, total // 2, total // 2 - 1}
    picks = {p for p in picks if 0 <= p < total}
    tiles = max(1, total // tile)
    for t in np.linspace(0, tiles - 1, num=min(tiles, want // 2), dtype=np.int64):
        picks.add(int(min(total - 1, t * tile + rng.integers(0, tile))))
    while len(picks) < want:
        picks.add(int(rng.integers(0, total)))
    return np.array(sorted(picks)[:want] if len(picks) > want else sorted(picks), dtype=np.int64)


def check_sample(plan: dict, inputs: Dict[str, np.ndarray], device_outputs: Dict[str, np.ndarray], units: Sequence[int],
                 lib=None) -> Dict[str, object]:
    """Compare the device's outputs on the sampled leading indices with the oracle's.

    ``inputs``: the full-batch graph inputs (integer codes); ``device_outputs``: name -> the device result ALREADY
    restricted to ``units`` (same order).  ``lib``: a C-oracle handle to evaluate with the C edition, None for the
    NumPy edition.  Returns {'rows_checked', 'values_checked', 'mismatches', 'oracle'}."""
    units = np.asarray(units, dtype=np.int64)
    sub = {k: np.ascontiguousarray(np.asarray(v)[units]) for k, v in inputs.items()}
    if lib is not None:
        want, _ = run_plan_c(lib, plan, sub)
    else:
        want = oracle.run_plan(plan, sub)
    mismatches = values = 0
    for name, ref in want.items():
        got = np.asarray(device_outputs[name])
        if got.shape != ref.shape:
            raise ValueError(f'{name}: device sample has shape {got.shape}, oracle {ref.shape}')
        mismatches += int((got.astype(np.int64) != ref.astype(np.int64)).sum())
        values += int(ref.size)
    return {'rows_checked': int(units.size), 'values_checked': values, 'mismatches': mismatches,
            'oracle': 'c' if lib is not None else 'numpy'}
