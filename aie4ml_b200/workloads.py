"""Seeded synthetic workloads: the five benchmark configurations as lowered-graph builders.

Each function returns ``(GraphBuilder, inputs)`` where ``inputs`` maps graph-input names to integer
code arrays drawn with ``numpy.random.default_rng(seed)``.  Constants are drawn as integer codes and
handed to the builder as ``code / 2**frac`` floats, which quantise back to exactly those codes.
The fixed-point labels (``frac``) are chosen so every layer's requantisation shift equals the value
the configuration names; labels do not change integer results, only the shifts they imply.
"""

from __future__ import annotations

from typing import Dict, Tuple

import numpy as np

from .frontends.graph import GraphBuilder, intent

Inputs = Dict[str, np.ndarray]

ROUNDING_BY_NAME = {'half_up': 'RND_HALF_UP', 'conv_even': 'RND_CONV', 'floor': 'TRN', 'sym_inf': 'RND'}


def _codes(rng, lo: int, hi: int, shape, dtype=np.int64) -> np.ndarray:
    return rng.integers(lo, hi + 1, size=shape, dtype=dtype)


def _gauss_table(sigma: float) -> np.ndarray:
    """65536-entry inverse-CDF table of clip(round(N(0, sigma^2)), -128, 127): entry u is the value whose
    cumulative probability interval contains (u + 0.5) / 65536."""
    import math

    cdf = np.array([0.5 * (1.0 + math.erf((v + 0.5) / (sigma * math.sqrt(2.0)))) for v in range(-128, 127)])
    q = (np.arange(65536, dtype=np.float64) + 0.5) / 65536.0
    return (np.searchsorted(cdf, q, side='right') - 128).astype(np.int8)


def _gauss_i8(rng, sigma: float, shape) -> np.ndarray:
    """int8 codes with a Gaussian profile (rounded, clipped to [-128, 127]): uniform 16-bit draws mapped through the
    inverse CDF of the discretised distribution.  A 2^30-element tensor takes seconds this way; drawing float
    normals and rounding them takes a minute."""
    table = _gauss_table(float(sigma))
    out = np.empty(shape, dtype=np.int8)
    flat = out.reshape(-1)
    step = 1 << 26
    for i in range(0, flat.size, step):
        n = min(step, flat.size - i)
        np.take(table, rng.integers(0, 65536, size=n, dtype=np.uint16), out=flat[i:i + n])
    return out


def _dense(b: GraphBuilder, rng, name: str, x: str, k: int, n: int, *, in_frac: int, out_frac: int, shift: int,
           w_lim: int, bias_lim, relu: bool, rnd: str, out_name=None, w_lo=None) -> str:
    """Dense whose resolved shift is ``shift``: the weight label is w.frac = out.frac + shift - in.frac."""
    w_frac = out_frac + shift - in_frac
    W = _codes(rng, -w_lim if w_lo is None else w_lo, w_lim, (k, n)).astype(np.float64) / float(1 << w_frac)
    bias = None
    if bias_lim is not None:
        bias = _codes(rng, -bias_lim, bias_lim, (n,)).astype(np.float64) / float(1 << (in_frac + w_frac))
    return b.dense(name, x, W, intent(8, w_frac, rounding=rnd), intent(8, out_frac, rounding=rnd), bias=bias,
                   bias_precision=intent(32, in_frac + w_frac, rounding=rnd) if bias is not None else None, relu=relu,
                   out_name=out_name)


def mlp_cfg1(batch: int = 1024, rounding: str = 'half_up', seed: int = 0) -> Tuple[GraphBuilder, Inputs]:
    """Int8 MLP 16->64->32->32->5, bias everywhere, ReLU on all but the last layer, shift 7."""
    rnd = ROUNDING_BY_NAME[rounding]
    rng = np.random.default_rng(seed)
    b = GraphBuilder({'Part': 'cuda_b200'}, name='mlp_cfg1')
    x = b.input('x', (batch, 16), intent(8, 4, rounding=rnd))
    dims = [16, 64, 32, 32, 5]
    cur = x
    for i in range(4):
        cur = _dense(b, rng, f'fc{i}', cur, dims[i], dims[i + 1], in_frac=4, out_frac=4, shift=7, w_lim=127,
                     bias_lim=1 << 12, relu=i < 3, rnd=rnd)
    b.output(cur)
    return b, {'x': _codes(rng, -128, 127, (batch, 16), np.int8)}


def dense_cfg2(M: int, K: int, N: int, rounding: str = 'half_up', seed: int = 1) -> Tuple[GraphBuilder, Inputs]:
    """Single int8 Dense with bias, shift 10, ReLU."""
    rnd = ROUNDING_BY_NAME[rounding]
    rng = np.random.default_rng(seed)
    b = GraphBuilder({'Part': 'cuda_b200'}, name='dense_cfg2')
    x = b.input('x', (M, K), intent(8, 4, rounding=rnd))
    y = _dense(b, rng, 'fc', x, K, N, in_frac=4, out_frac=4, shift=10, w_lim=127, bias_lim=1 << 16, relu=True, rnd=rnd,
               w_lo=-128)
    b.output(y)
    return b, {'x': _codes(rng, -128, 127, (M, K), np.int8)}


def encoder_cfg3(batch: int = 4096, softmax: str = 'exp', rounding: str = 'half_up', seed: int = 2,
                 seq: int = 128, d_model: int = 256, heads: int = 4, ffn: int = 1024) -> Tuple[GraphBuilder, Inputs]:
    """Int8 transformer encoder block: QKV/O/FFN Dense, per-head QK^T and AV dynamic MatMul, quantized
    Softmax (``exp`` accurate or ``hccs`` surrogate), two residual Adds, two LayerNorms, head split and
    merge through Split / Transpose / Concat views."""
    rnd = ROUNDING_BY_NAME[rounding]
    rng = np.random.default_rng(seed)
    dh = d_model // heads
    directives = {}
    if softmax == 'hccs':
        directives = {f'sm{h}': {'approximation': 'hccs', 'hccs': {'B': 200, 'S': 3, 'Dmax': 66}} for h in range(heads)}
    b = GraphBuilder({'Part': 'cuda_b200', 'LayerDirectives': directives}, name=f'encoder_cfg3_{softmax}')
    XF, QF, SF, PF = 6, 5, 1, 8  # fixed-point labels: input, q/k/v, scores, probabilities
    x = b.input('x', (batch, seq, d_model), intent(8, XF, rounding=rnd))
    q = _dense(b, rng, 'wq', x, d_model, d_model, in_frac=XF, out_frac=QF, shift=8, w_lim=64, bias_lim=None,
               relu=False, rnd=rnd)
    k = _dense(b, rng, 'wk', x, d_model, d_model, in_frac=XF, out_frac=QF, shift=8, w_lim=64, bias_lim=None,
               relu=False, rnd=rnd)
    v = _dense(b, rng, 'wv', x, d_model, d_model, in_frac=XF, out_frac=QF, shift=8, w_lim=64, bias_lim=None,
               relu=False, rnd=rnd)
    qs = b.split('split_q', q, [dh] * heads, axis=-1)
    ks = b.split('split_k', k, [dh] * heads, axis=-1)
    vs = b.split('split_v', v, [dh] * heads, axis=-1)
    ctx_heads = []
    for h in range(heads):
        kt = b.transpose(f'kt{h}', ks[h], [0, 2, 1])
        s = b.matmul(f'qk{h}', qs[h], kt, intent(8, SF, rounding=rnd))         # shift 2*QF - SF = 9
        if softmax == 'exp':
            s = b.scale(f'scale{h}', s, 1.0 / np.sqrt(float(dh)))                 # -> softmax temperature
        p = b.softmax(f'sm{h}', s, intent(8, PF, signed=False, rounding=rnd))
        ctx_heads.append(b.matmul(f'av{h}', p, vs[h], intent(8, QF, rounding=rnd)))  # shift PF = 8
    merged = b.concat('merge', ctx_heads, axis=-1)
    o = _dense(b, rng, 'wo', merged, d_model, d_model, in_frac=QF, out_frac=XF, shift=9, w_lim=64, bias_lim=None,
               relu=False, rnd=rnd)
    r1 = b.add('res1', x, o, intent(8, XF, rounding=rnd))
    LF = 4
    g1 = _codes(rng, -256, 256, (d_model,)).astype(np.float64) / 128.0
    b1 = _codes(rng, -256, 256, (d_model,)).astype(np.float64) / 32768.0
    n1 = b.layer_norm('ln1', r1, g1, b1, intent(8, LF, rounding=rnd), eps_q0=1)
    f1 = _dense(b, rng, 'ffn1', n1, d_model, ffn, in_frac=LF, out_frac=LF, shift=8, w_lim=64, bias_lim=None,
                relu=True, rnd=rnd)
    f2 = _dense(b, rng, 'ffn2', f1, ffn, d_model, in_frac=LF, out_frac=LF, shift=9, w_lim=64, bias_lim=None,
                relu=False, rnd=rnd)
    r2 = b.add('res2', n1, f2, intent(8, LF, rounding=rnd))
    g2 = _codes(rng, -256, 256, (d_model,)).astype(np.float64) / 128.0
    b2 = _codes(rng, -256, 256, (d_model,)).astype(np.float64) / 32768.0
    y = b.layer_norm('ln2', r2, g2, b2, intent(8, LF, rounding=rnd), eps_q0=1)
    b.output(y)
    return b, {'x': _gauss_i8(rng, 24.0, (batch, seq, d_model))}


def rowops_cfg4(rows: int = 1 << 20, cols: int = 1024, op: str = 'layer_norm', rounding: str = 'half_up',
                seed: int = 3) -> Tuple[GraphBuilder, Inputs]:
    """A bandwidth-bound row op (``layer_norm``, ``softmax_exp`` or ``softmax_hccs``) followed by an
    Elementwise Add with a second random tensor of the row op's output type."""
    rnd = ROUNDING_BY_NAME[rounding]
    rng = np.random.default_rng(seed)
    directives = {}
    if op == 'softmax_hccs':
        directives = {'sm': {'approximation': 'hccs', 'hccs': {'B': 31, 'S': 1, 'Dmax': 30}}}
    b = GraphBuilder({'Part': 'cuda_b200', 'LayerDirectives': directives}, name=f'rowops_cfg4_{op}')
    x = b.input('x', (rows, cols), intent(8, 4, rounding=rnd))
    inputs: Inputs = {}
    gamma = _codes(rng, -256, 256, (cols,)).astype(np.float64) / 128.0
    beta = _codes(rng, -256, 256, (cols,)).astype(np.float64) / 32768.0
    inputs['x'] = _gauss_i8(rng, 32.0, (rows, cols))
    if op == 'layer_norm':
        out_p = intent(8, 4, rounding=rnd)
        mid = b.layer_norm('ln', x, gamma, beta, out_p, eps_q0=1)
        inputs['r'] = _codes(rng, -128, 127, (rows, cols), np.int8)
    elif op in ('softmax_exp', 'softmax_hccs'):
        out_p = intent(8, 8, signed=False, rounding=rnd)
        mid = b.softmax('sm', x, out_p)
        inputs['r'] = _codes(rng, 0, 255, (rows, cols), np.uint8)
    else:
        raise ValueError(f'unknown row op {op!r}')
    r = b.input('r', (rows, cols), out_p)
    y = b.add('add', mid, r, out_p)
    b.output(y)
    return b, inputs


def wide_mlp_cfg5(batch: int = 262144, rounding: str = 'half_up', seed: int = 4) -> Tuple[GraphBuilder, Inputs]:
    """Input 512 fans out to two branches of four 1024-wide Dense+ReLU layers, Concat to 2048,
    Dense 2048->1024 (ReLU) -> 10; bias everywhere, shift 9."""
    rnd = ROUNDING_BY_NAME[rounding]
    rng = np.random.default_rng(seed)
    b = GraphBuilder({'Part': 'cuda_b200'}, name='wide_mlp_cfg5')
    x = b.input('x', (batch, 512), intent(8, 4, rounding=rnd))
    branches = []
    for br in range(2):
        cur, k = x, 512
        for i in range(4):
            cur = _dense(b, rng, f'b{br}_fc{i}', cur, k, 1024, in_frac=4, out_frac=4, shift=9, w_lim=127,
                         bias_lim=1 << 14, relu=True, rnd=rnd)
            k = 1024
        branches.append(cur)
    cat = b.concat('cat', branches, axis=-1)
    h = _dense(b, rng, 'head0', cat, 2048, 1024, in_frac=4, out_frac=4, shift=9, w_lim=127, bias_lim=1 << 14,
               relu=True, rnd=rnd)
    y = _dense(b, rng, 'head1', h, 1024, 10, in_frac=4, out_frac=4, shift=9, w_lim=127, bias_lim=1 << 14, relu=False,
               rnd=rnd)
    b.output(y)
    return b, {'x': _codes(rng, -128, 127, (batch, 512), np.int8)}
