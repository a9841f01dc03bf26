"""Benchmark configurations written as ONNX Q/DQ graphs (neutral ``OnnxGraph`` descriptions, no ``onnx`` package
needed): the patterns the reference importer accepts (``src/aie4ml/frontends/onnx/quantize.py:35-135``,
``handlers/matmul.py:16-137``, ``handlers/tensor.py:16-163``) -- an integer graph input fed straight into a
DequantizeLinear or a float input through QuantizeLinear -> DequantizeLinear, weights as DequantizeLinear of an int8
initializer, Gemm bias as DequantizeLinear of an int32 initializer at scale s_x * s_w, a Q/DQ pair on every
activation edge, Mul(1/sqrt(d)) in front of Softmax, Split / Transpose / Concat for the heads, LayerNormalization with
float Scale / B, ``LayerDirectives`` for the surrogate softmax.  Test infrastructure."""

import numpy as np

from aie4ml_b200.frontends.onnx_import import OnnxGraph, OnnxNode


class _G:
    def __init__(self):
        self.nodes, self.inits = [], {}

    def qdq(self, src, name, frac, dtype=np.int8):
        """src -> QuantizeLinear -> DequantizeLinear; returns the DQ output name."""
        self.inits[f'{name}_s'] = np.array(2.0 ** -frac, dtype=np.float32)
        self.inits[f'{name}_z'] = np.array(0, dtype=dtype)
        self.nodes.append(OnnxNode('QuantizeLinear', f'{name}_q', [src, f'{name}_s', f'{name}_z'], [f'{name}_qo']))
        self.nodes.append(OnnxNode('DequantizeLinear', f'{name}_dq', [f'{name}_qo', f'{name}_s', f'{name}_z'], [f'{name}_dqo']))
        return f'{name}_dqo'

    def dq(self, src, name, frac, dtype):
        """DequantizeLinear of an integer graph input or initializer `src`."""
        self.inits[f'{name}_s'] = np.array(2.0 ** -frac, dtype=np.float32)
        self.inits[f'{name}_z'] = np.array(0, dtype=dtype)
        self.nodes.append(OnnxNode('DequantizeLinear', f'{name}_dq', [src, f'{name}_s', f'{name}_z'], [f'{name}_f']))
        return f'{name}_f'

    def const(self, name, codes, frac):
        self.inits[name] = codes
        return self.dq(name, name, frac, codes.dtype)

    def node(self, op, name, inputs, outputs, **attrs):
        self.nodes.append(OnnxNode(op, name, list(inputs), list(outputs), attrs))
        return outputs[0]


def mlp_cfg1_onnx(batch=1024, seed=0, float_input=False):
    """Int8 MLP 16->64->32->32->5 (Gemm with int32 bias, ReLU on all but the last layer, requantisation shift 7).
    -> (OnnxGraph, inputs): integer codes for the int8 graph input, or floats in [-1, 1) when `float_input`."""
    rng = np.random.default_rng(seed)
    g = _G()
    dims = [16, 64, 32, 32, 5]
    XF = 4
    if float_input:
        cur = g.qdq('x', 'xin', XF)
        inputs = {'x': ((batch, 16), np.float32)}
        x = (rng.random((batch, 16), dtype=np.float32) * 2.0) - 1.0
    else:
        cur = g.dq('x', 'xin', XF, np.int8)
        inputs = {'x': ((batch, 16), np.int8)}
        x = rng.integers(-128, 128, (batch, 16)).astype(np.int8)
    for i in range(4):
        w = rng.integers(-127, 128, (dims[i], dims[i + 1])).astype(np.int8)
        b = rng.integers(-(1 << 12), (1 << 12) + 1, dims[i + 1]).astype(np.int32)
        w_frac = XF + 7 - XF                       # shift = x.frac + w.frac - out.frac = 7
        y = g.node('Gemm', f'fc{i}', [cur, g.const(f'w{i}', w, w_frac), g.const(f'b{i}', b, XF + w_frac)], [f'fc{i}_o'])
        if i < 3:
            y = g.node('Relu', f'act{i}', [y], [f'act{i}_o'])
        cur = g.qdq(y, f'h{i}', XF)
    return OnnxGraph(g.nodes, g.inits, inputs, [cur], 'mlp_cfg1_onnx'), {'x': x}


def encoder_cfg3_onnx(batch=4, softmax='exp', seed=2, seq=128, d_model=256, heads=4, ffn=1024):
    """Int8 transformer encoder block as a Q/DQ graph -> (OnnxGraph, inputs, config).  `config` carries the
    LayerDirectives of the surrogate softmax when softmax == 'hccs' (there is then no Mul in front of the Softmax:
    the surrogate takes no temperature)."""
    rng = np.random.default_rng(seed)
    g = _G()
    dh = d_model // heads
    XF, QF, SF, PF, LF = 6, 5, 1, 8, 4
    x = g.dq('x', 'xin', XF, np.int8)

    def dense(name, src, k, n, in_frac, out_frac, shift, relu=False):
        w = rng.integers(-64, 65, (k, n)).astype(np.int8)
        y = g.node('MatMul', name, [src, g.const(f'{name}_w', w, out_frac + shift - in_frac)], [f'{name}_o'])
        if relu:
            y = g.node('Relu', f'{name}_relu', [y], [f'{name}_relu_o'])
        return g.qdq(y, f'{name}_act', out_frac)

    q = dense('wq', x, d_model, d_model, XF, QF, 8)
    k = dense('wk', x, d_model, d_model, XF, QF, 8)
    v = dense('wv', x, d_model, d_model, XF, QF, 8)
    g.inits['head_sizes'] = np.array([dh] * heads, dtype=np.int64)
    qs = [f'q{h}' for h in range(heads)]
    ks = [f'k{h}' for h in range(heads)]
    vs = [f'v{h}' for h in range(heads)]
    g.node('Split', 'split_q', [q, 'head_sizes'], qs, axis=-1)
    g.node('Split', 'split_k', [k, 'head_sizes'], ks, axis=-1)
    g.node('Split', 'split_v', [v, 'head_sizes'], vs, axis=-1)
    g.inits['inv_sqrt_d'] = np.array(1.0 / np.sqrt(float(dh)), dtype=np.float32)
    ctx = []
    directives = {}
    for h in range(heads):
        kt = g.node('Transpose', f'kt{h}', [ks[h]], [f'kt{h}_o'], perm=[0, 2, 1])
        s = g.qdq(g.node('MatMul', f'qk{h}', [qs[h], kt], [f'qk{h}_o']), f's{h}', SF)
        if softmax == 'exp':
            s = g.node('Mul', f'scale{h}', [s, 'inv_sqrt_d'], [f'scale{h}_o'])
        else:
            directives[f'sm{h}'] = {'approximation': 'hccs', 'hccs': {'B': 200, 'S': 3, 'Dmax': 66}}
        p = g.qdq(g.node('Softmax', f'sm{h}', [s], [f'sm{h}_o'], axis=-1), f'p{h}', PF, np.uint8)
        ctx.append(g.qdq(g.node('MatMul', f'av{h}', [p, vs[h]], [f'av{h}_o']), f'c{h}', QF))
    merged = g.node('Concat', 'merge', ctx, ['merge_o'], axis=-1)
    o = dense('wo', merged, d_model, d_model, QF, XF, 9)
    r1 = g.qdq(g.node('Add', 'res1', [x, o], ['res1_o']), 'r1', XF)
    g.inits['g1'] = (rng.integers(-256, 257, d_model) / 128.0).astype(np.float32)
    g.inits['b1'] = (rng.integers(-256, 257, d_model) / 32768.0).astype(np.float32)
    n1 = g.qdq(g.node('LayerNormalization', 'ln1', [r1, 'g1', 'b1'], ['ln1_o'], axis=-1, epsilon=2.0 ** (-2 * XF)), 'n1', LF)
    f1 = dense('ffn1', n1, d_model, ffn, LF, LF, 8, relu=True)
    f2 = dense('ffn2', f1, ffn, d_model, LF, LF, 9)
    r2 = g.qdq(g.node('Add', 'res2', [n1, f2], ['res2_o']), 'r2', LF)
    g.inits['g2'] = (rng.integers(-256, 257, d_model) / 128.0).astype(np.float32)
    g.inits['b2'] = (rng.integers(-256, 257, d_model) / 32768.0).astype(np.float32)
    y = g.qdq(g.node('LayerNormalization', 'ln2', [r2, 'g2', 'b2'], ['ln2_o'], axis=-1, epsilon=2.0 ** (-2 * LF)), 'y', LF)
    xin = np.clip(np.rint(rng.standard_normal((batch, seq, d_model)) * 24.0), -128, 127).astype(np.int8)
    config = {'Part': 'cuda_b200', 'LayerDirectives': directives}
    return OnnxGraph(g.nodes, g.inits, {'x': ((batch, seq, d_model), np.int8)}, [y], f'encoder_cfg3_onnx_{softmax}'), {'x': xin}, config


BUILTIN = {
    'mlp_cfg1': lambda batch, seed: mlp_cfg1_onnx(batch, seed) + ({'Part': 'cuda_b200'},),
    'mlp_cfg1_float': lambda batch, seed: mlp_cfg1_onnx(batch, seed, float_input=True) + ({'Part': 'cuda_b200'},),
    'encoder_exp': lambda batch, seed: encoder_cfg3_onnx(batch, 'exp', seed),
    'encoder_hccs': lambda batch, seed: encoder_cfg3_onnx(batch, 'hccs', seed),
}
