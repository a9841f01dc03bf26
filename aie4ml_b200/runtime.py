"""The CUDA runtime that replaces the reference's AIE emitter / placement / simulator tail.

It walks the lowered IR (logical nodes + execution entries produced by Resolve / Pack) and
builds a *plan*: one HBM buffer per stored tensor, zero-copy views for Split / Slice / Concat /
fanout / transposed operands (the reference realises those as memory-tile DMA descriptors,
``src/aie4ml/passes/fold_views.py:69-150`` and ``passes/transport/*``), and an ordered list of
kernel launches through the C ABI.  A row op followed by an exact-type Add is fused into one
launch when the intermediate has no other consumer (the analogue of the reference's "direct"
neighbour transport, ``passes/transport/classify.py:25-49``).

PyTorch is used only for device memory, streams and CUDA-graph capture.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple

import numpy as np

from . import lib as _lib
from .ir import BackendContext, input_tensor_for_role
from .op_impls.precision import DTYPE_CODE, FLOAT_CODE, ROUNDING_CODE, resolve_exact_storage_dtype

ESZ = {'int8': 1, 'uint8': 1, 'int16': 2, 'int32': 4, 'bfloat16': 2, 'float32': 4, 'fp8_e4m3': 1}
NP_DT = {'int8': np.int8, 'uint8': np.uint8, 'int16': np.int16, 'int32': np.int32, 'bfloat16': np.uint16,
         'float32': np.float32, 'fp8_e4m3': np.uint8}


def _torch():
    import torch

    return torch


@dataclass(frozen=True)
class View:
    """A strided window into a root buffer.  Offsets and strides in elements."""

    root: str
    offset: int
    shape: Tuple[int, ...]
    strides: Tuple[int, ...]
    fmt: str

    @property
    def esz(self) -> int:
        return ESZ[self.fmt]


def padded_pitch(cols: int, esz: int) -> int:
    """Row pitch in elements so that every row starts on a 16-byte boundary (TMA and 128-bit
    accesses need that; e.g. a 5- or 10-wide int8 output gets pitch 16)."""
    return (cols * esz + 15) // 16 * 16 // esz


def contiguous_strides(shape: Sequence[int], esz: int) -> Tuple[int, ...]:
    if not shape:
        return ()
    strides = [1] * len(shape)
    pitch = padded_pitch(int(shape[-1]), esz)
    acc = pitch
    for i in range(len(shape) - 2, -1, -1):
        strides[i] = acc
        acc *= int(shape[i])
    return tuple(strides)


def collapse_2d(view: View, what: str) -> Tuple[int, int, int, int]:
    """(element offset, rows, cols, pitch) of a view whose leading axes fold into rows."""
    shape, strides = view.shape, view.strides
    if strides[-1] != 1:
        raise NotImplementedError(f'{what}: last axis must be contiguous.')
    cols = int(shape[-1])
    if len(shape) == 1:
        return view.offset, 1, cols, cols
    lead = [(int(s), int(st)) for s, st in zip(shape[:-1], strides[:-1]) if int(s) != 1]
    if not lead:
        return view.offset, 1, cols, max(cols, int(strides[-2]))
    for (_, st_outer), (s_inner, st_inner) in zip(lead[:-1], lead[1:]):
        if st_outer != st_inner * s_inner:
            raise NotImplementedError(f'{what}: leading axes of the view do not fold into uniform rows '
                                      f'(shape {shape}, strides {strides}).')
    rows = 1
    for s, _ in lead:
        rows *= s
    return view.offset, rows, cols, lead[-1][1]


def collapse_batched(view: View, what: str) -> Tuple[int, int, int, int, int, int]:
    """(offset, batch, rows, cols, pitch, batch stride) of a stack of matrices."""
    shape, strides = view.shape, view.strides
    if len(shape) < 2 or strides[-1] != 1:
        raise NotImplementedError(f'{what}: expected a stack of row-major matrices.')
    rows, cols, pitch = int(shape[-2]), int(shape[-1]), int(strides[-2])
    lead = [(int(s), int(st)) for s, st in zip(shape[:-2], strides[:-2]) if int(s) != 1]
    if not lead:
        return view.offset, 1, rows, cols, pitch, 0
    for (_, st_outer), (s_inner, st_inner) in zip(lead[:-1], lead[1:]):
        if st_outer != st_inner * s_inner:
            raise NotImplementedError(f'{what}: batch axes of the view do not fold into one stride '
                                      f'(shape {shape}, strides {strides}).')
    batch = 1
    for s, _ in lead:
        batch *= s
    return view.offset, batch, rows, cols, pitch, lead[-1][1]


class Plan:
    """Buffers, views, device constants and the launch list of one lowered model."""

    def __init__(self, ctx: BackendContext, device: Optional[str] = None, fuse_rowop_add: bool = True,
                 dense_algo: int = _lib.ALGO_AUTO, share_params: Optional['Plan'] = None, fuse_attention: bool = True,
                 fuse_dense_chain: bool = True, merge_attention_heads: bool = True, merge_parallel_dense: bool = True,
                 fuse_dense_ln: bool = True):
        torch = _torch()
        self.ctx = ctx
        self.lib = _lib.load()
        if not torch.cuda.is_available():
            raise RuntimeError('aie4ml_b200 executes on a CUDA device only; no GPU is visible and there is no '
                               'CPU execution path.')
        self.device = torch.device(device or f'cuda:{torch.cuda.current_device()}')
        # The C ABI works on the CURRENT device (status word, SM count, scratch, shared-memory opt-in), so every
        # entry into it from this plan runs with the plan's device current, whatever the caller had selected.
        with torch.cuda.device(self.device):
            self._build(ctx, fuse_rowop_add, dense_algo, share_params, fuse_attention, fuse_dense_chain,
                        merge_attention_heads, merge_parallel_dense, fuse_dense_ln)

    def _build(self, ctx, fuse_rowop_add, dense_algo, share_params, fuse_attention, fuse_dense_chain,
               merge_attention_heads, merge_parallel_dense, fuse_dense_ln) -> None:
        torch = _torch()
        self.dense_algo = int(dense_algo)
        self.fuse_rowop_add = bool(fuse_rowop_add)
        self.fuse_attention = bool(fuse_attention)
        self.merge_attention_heads = bool(merge_attention_heads)
        self.merge_parallel_dense = bool(merge_parallel_dense)
        self.fuse_dense_chain = bool(fuse_dense_chain)
        graph = ctx.ir.logical
        self.graph = graph

        # 1. storage format of every activation tensor
        self.fmt: Dict[str, str] = {}
        for name, t in graph.tensors.items():
            if t.is_parameter:
                continue
            self.fmt[name] = resolve_exact_storage_dtype(t.precision, namespace='tensor', layer_name=name).format
            if self.fmt[name] not in ('int8', 'uint8', 'int16', 'bfloat16', 'float32', 'fp8_e4m3'):
                raise NotImplementedError(f'{name}: activation format {self.fmt[name]!r} has no kernel.')

        # 2. aliases introduced by view placeholders
        self.alias: Dict[str, Tuple[str, int, int]] = {}
        for node in graph.nodes:
            if not node.is_placeholder:
                continue
            if 'concat_view' in node.traits:
                data = node.traits['concat_view'].data
                for piece in data['slices']:
                    self._add_alias(piece['input'], data['output'], int(data['axis']), int(piece['start']), node.name)
            elif 'slice_view' in node.traits:
                data = node.traits['slice_view'].data
                for piece in data['slices']:
                    self._add_alias(piece['output'], data['source'], int(data['axis']), int(piece['start']), node.name)
            else:
                raise NotImplementedError(f'{node.name}: placeholder without a view trait.')

        # 3. logical op list (dicts), fusion, then roots and views
        self.ops: List[Dict[str, Any]] = []
        self.params_np: Dict[str, np.ndarray] = {}
        for node in graph.nodes:
            if node.is_placeholder:
                continue
            inst = ctx.ir.execution.get(node.name)
            if inst is None:
                raise RuntimeError(f'{node.name}: not resolved; run the pass pipeline first.')
            op = inst.variant.plan_op(inst)
            if op['kind'] in ('dense', 'dense_f'):
                self.params_np[op['weight']] = inst.artifacts['packed_weights']
                if op['bias']:
                    self.params_np[op['bias']] = inst.artifacts['packed_bias']
            elif op['kind'] == 'layer_norm':
                self.params_np[op['gamma']] = inst.artifacts['packed_gamma']
                self.params_np[op['beta']] = inst.artifacts['packed_beta']
            elif op['kind'] in ('matmul', 'matmul_f'):
                if input_tensor_for_role(node, 'rhs').is_parameter:
                    raise NotImplementedError(f'{node.name}: a constant RHS of rank > 2 has no kernel; '
                                              'express it as dense.')
            self.ops.append(op)
        self.fused: List[str] = []
        self.views: Dict[str, View] = {}
        self.buffers: Dict[str, Any] = {}
        self.synthetic: Dict[str, Tuple[int, ...]] = {}     # tensors the plan adds (name -> shape): merged outputs
        if merge_parallel_dense:
            self._merge_parallel_dense()
        if fuse_attention:
            self._fuse_attention()
            if merge_attention_heads:
                self._merge_attention_heads()
        self._keepalive: List[Any] = []
        if fuse_dense_chain:
            self._fuse_dense_chain()
        if fuse_rowop_add:
            self._fuse_add_layernorm()
            if fuse_dense_ln:
                self._fuse_dense_add_layernorm()
            self._fuse_rowop_add()

        live = set(graph.input_tensor_names) | set(graph.output_tensor_names)
        for op in self.ops:
            for key in ('lhs', 'rhs', 'out', 'addend', 'pre_addend', 'residual', 'q', 'k', 'v'):
                if op.get(key):
                    live.add(op[key])
            for member in op.get('members', ()):
                live.update(member.values())
        for name in sorted(live):
            self._view(name)

        # 4. device constants
        #    (a second plan of the same model on the same device reuses the first one's constants)
        self.params: Dict[str, Any] = {}
        if share_params is not None:
            if share_params.device != self.device or set(share_params.params) != set(self.params_np):
                raise ValueError('share_params: the other plan holds different constants or lives on another device.')
            self.params = share_params.params
        else:
            for key, arr in self.params_np.items():
                self.params[key] = torch.from_numpy(np.ascontiguousarray(arr)).to(self.device)

        # 5. launches
        self.launches: List[Tuple[Callable, tuple]] = []
        for op in self.ops:
            self.launches.append(self._compile(op))
        self.graph_exec = None

    # ---- views ---------------------------------------------------------------------------------
    def _add_alias(self, child: str, parent: str, axis: int, start: int, node_name: str) -> None:
        if child in self.alias:
            raise NotImplementedError(f'{node_name}: tensor {child!r} would need two storage locations '
                                      '(chained or overlapping view ops); insert a copy in the model.')
        self.alias[child] = (parent, axis, start)

    def _view(self, name: str) -> View:
        if name in self.views:
            return self.views[name]
        torch = _torch()
        fmt = self.fmt[name]
        shape = self.synthetic[name] if name in self.synthetic else tuple(int(s) for s in self.graph.tensors[name].shape)
        if name in self.alias:
            parent, axis, start = self.alias[name]
            pv = self._view(parent)
            if pv.fmt != fmt:
                raise ValueError(f'{name}: view of {parent!r} changes the storage type ({pv.fmt} -> {fmt}).')
            view = View(root=pv.root, offset=pv.offset + start * pv.strides[axis], shape=shape, strides=pv.strides,
                        fmt=fmt)
        else:
            strides = contiguous_strides(shape, ESZ[fmt])
            total = (shape[0] * strides[0]) if shape else 1
            self.buffers[name] = torch.zeros(total * ESZ[fmt], dtype=torch.uint8, device=self.device)
            view = View(root=name, offset=0, shape=shape, strides=strides, fmt=fmt)
        self.views[name] = view
        return view

    def ptr(self, view: View, offset: Optional[int] = None) -> int:
        off = view.offset if offset is None else offset
        return self.buffers[view.root].data_ptr() + off * view.esz

    def tensor_of(self, name: str):
        """A torch tensor (strided) over the view's storage, typed by the tensor's format."""
        torch = _torch()
        v = self._view(name)
        dt = {'int8': torch.int8, 'uint8': torch.uint8, 'int16': torch.int16, 'bfloat16': torch.bfloat16,
              'float32': torch.float32, 'fp8_e4m3': torch.float8_e4m3fn}[v.fmt]
        base = self.buffers[v.root].view(dt)
        return base.as_strided(v.shape, v.strides, v.offset)

    # ---- fusion --------------------------------------------------------------------------------
    def _fuse_rowop_add(self) -> None:
        """layer_norm/softmax -> add (same type, shift 0) becomes one launch when the row op's output
        feeds nothing else, is not a graph output or a view, and the other addend already exists."""
        graph = self.graph
        produced_at = {op['out']: i for i, op in enumerate(self.ops)}
        aliased = set(self.alias) | {p for p, _, _ in self.alias.values()}
        drop = set()
        for i, op in enumerate(self.ops):
            if op['kind'] != 'add' or op['shift'] != 0:
                continue
            for mid_key, other_key in (('lhs', 'rhs'), ('rhs', 'lhs')):
                mid, other = op[mid_key], op[other_key]
                j = produced_at.get(mid)
                if j is None or j in drop:
                    continue
                prod = self.ops[j]
                if prod['kind'] not in ('layer_norm', 'softmax') or prod.get('addend') or prod.get('pre_addend'):
                    continue
                t = graph.tensors[mid]
                if len(t.consumers) != 1 or mid in graph.output_tensor_names or mid in aliased:
                    continue
                if produced_at.get(other, -1) > j:  # addend must exist when the row op runs
                    continue
                if self.fmt[mid] != self.fmt[op['out']] or self.fmt[other] != self.fmt[mid]:
                    continue
                prod['addend'] = other
                prod['fused_out'] = op['out']
                self.fused.append(f"{prod['name']}+{op['name']}")
                drop.add(i)
                break
        if drop:
            for op in self.ops:
                if op.get('fused_out'):
                    op['out'] = op.pop('fused_out')
            self.ops = [op for i, op in enumerate(self.ops) if i not in drop]

    def _merge_parallel_dense(self) -> None:
        """Dense layers that read the same tensor with the same requantisation (the Q / K / V projections of an
        attention layer) become ONE Dense over the concatenated weights: the input is read once, and the outputs
        become column slices of one wider tensor.  Each output must own its storage so far (not a view, not a
        graph output) and be a whole number of 16-byte pieces wide."""
        graph = self.graph
        groups: Dict[tuple, List[int]] = {}
        for i, op in enumerate(self.ops):
            if (op['kind'] != 'dense' or op['transpose_lhs'] or op['lhs_dtype'] not in ('int8', 'uint8')
                    or op.get('rhs_dtype', 'int8') != 'int8' or op['out_dtype'] not in ('int8', 'uint8')):
                continue
            out = op['out']
            if out in self.alias or out in graph.output_tensor_names or op['N'] % 16:
                continue
            lead = tuple(int(d) for d in graph.tensors[out].shape[:-1])
            key = (op['lhs'], op['K'], op['shift'], op['rounding'], op['relu'], op['out_dtype'], op['lhs_dtype'], lead)
            groups.setdefault(key, []).append(i)
        replace, drop = {}, set()
        for key, members in groups.items():
            if len(members) < 2:
                continue
            layers = [self.ops[i] for i in members]
            lead = key[-1]
            total = sum(l['N'] for l in layers)
            name = '|'.join(l['out'] for l in layers)
            self.synthetic[name] = lead + (total,)
            self.fmt[name] = self.fmt[layers[0]['out']]
            start = 0
            for l in layers:
                self._add_alias(l['out'], name, len(lead), start, l['name'])
                start += l['N']
            merged_name = '|'.join(l['name'] for l in layers)
            weight = f'{merged_name}/weights'
            self.params_np[weight] = np.concatenate([self.params_np.pop(l['weight']) for l in layers], axis=0)
            bias = None
            if any(l['bias'] for l in layers):
                bias = f'{merged_name}/bias'
                self.params_np[bias] = np.concatenate(
                    [self.params_np.pop(l['bias']) if l['bias'] else np.zeros(l['N'], dtype=np.int32) for l in layers])
            # at the first member's place: the shared input exists there, and no output is needed any earlier
            replace[members[0]] = dict(layers[0], name=merged_name, out=name, N=total, weight=weight, bias=bias)
            drop.update(members[1:])
            self.fused.append(merged_name)
        if replace:
            self.ops = [replace.get(i, op) for i, op in enumerate(self.ops) if i not in drop]

    def _fuse_dense_chain(self) -> None:
        """Consecutive Dense layers whose intermediates feed nothing else become one `mlp` op when the library
        runs such a chain as a single kernel (a4c_mlp_i8_single_kernel): weights and activations then stay in
        shared memory and the intermediates get no buffer."""
        import ctypes

        graph = self.graph
        aliased = set(self.alias) | {p for p, _, _ in self.alias.values()}
        consumer_of = {}
        for i, op in enumerate(self.ops):
            for key in ('lhs', 'rhs'):
                if op.get(key):
                    consumer_of.setdefault(op[key], []).append(i)

        def chainable(op) -> bool:
            return (op['kind'] == 'dense' and not op['transpose_lhs'] and op['lhs_dtype'] in ('int8', 'uint8')
                    and op.get('rhs_dtype', 'int8') == 'int8')

        used, chains = set(), []
        for i, op in enumerate(self.ops):
            if i in used or not chainable(op):
                continue
            chain = [i]
            while True:
                cur = self.ops[chain[-1]]
                mid = cur['out']
                nxt = consumer_of.get(mid, [])
                if (len(nxt) != 1 or len(graph.tensors[mid].consumers) != 1 or mid in graph.output_tensor_names
                        or mid in aliased or self.fmt[mid] != 'int8' or cur['out_dtype'] != 'int8'):
                    break
                j = nxt[0]
                cand = self.ops[j]
                if (j in used or not chainable(cand) or cand['lhs'] != mid or cand['rounding'] != op['rounding']
                        or j != chain[-1] + 1):
                    break
                chain.append(j)
            if len(chain) < 2:
                continue
            layers = [self.ops[j] for j in chain]
            dims = [layers[0]['K']] + [l['N'] for l in layers]
            rows = int(np.prod(graph.tensors[layers[0]['lhs']].shape[:-1]))
            arr = (ctypes.c_int * len(dims))(*dims)
            if not self.lib.a4c_mlp_i8_single_kernel(len(layers), arr, DTYPE_CODE[layers[-1]['out_dtype']], rows):
                continue
            chains.append((chain, layers, dims))
            used.update(chain)
        if not chains:
            return
        replace, drop = {}, set()
        for chain, layers, dims in chains:
            name = '+'.join(l['name'] for l in layers)
            replace[chain[-1]] = {'kind': 'mlp', 'name': name, 'lhs': layers[0]['lhs'], 'out': layers[-1]['out'],
                                  'layers': layers, 'dims': dims, 'rounding': layers[0]['rounding']}
            drop.update(chain[:-1])
            self.fused.append(name)
        self.ops = [replace.get(i, op) for i, op in enumerate(self.ops) if i not in drop]

    def _fuse_add_layernorm(self) -> None:
        """add (same int8 type, shift 0) -> layer_norm becomes one launch that adds while it loads: the sum is
        never stored.  The sum must feed only the LayerNorm and be neither a graph output nor a view."""
        graph = self.graph
        produced_at = {op['out']: i for i, op in enumerate(self.ops)}
        aliased = set(self.alias) | {p for p, _, _ in self.alias.values()}
        drop = set()
        for ln in self.ops:
            if ln['kind'] != 'layer_norm' or ln.get('addend'):
                continue
            mid = ln['lhs']
            j = produced_at.get(mid)
            if j is None or j in drop:
                continue
            add = self.ops[j]
            if add['kind'] != 'add' or add['shift'] != 0:
                continue
            if len(graph.tensors[mid].consumers) != 1 or mid in graph.output_tensor_names or mid in aliased:
                continue
            if any(self.fmt[t] != 'int8' for t in (add['lhs'], add['rhs'], mid)):
                continue
            ln['lhs'], ln['pre_addend'] = add['lhs'], add['rhs']
            self.fused.append(f"{add['name']}+{ln['name']}")
            drop.add(j)
        if drop:
            self.ops = [op for i, op in enumerate(self.ops) if i not in drop]

    def _fuse_dense_add_layernorm(self) -> None:
        """dense -> add (residual) -> layer_norm becomes one launch when the library has the single kernel for the
        shapes (a4c_dense_add_layernorm_supported: the layer is 256 features wide, so one accumulator tile holds whole
        rows).  Runs after the Add has been folded into the LayerNorm; the Dense output must feed only that Add and be
        neither a graph output nor a view.  Neither the Dense output nor the sum gets a buffer."""
        graph = self.graph
        produced_at = {op['out']: i for i, op in enumerate(self.ops)}
        aliased = set(self.alias) | {p for p, _, _ in self.alias.values()}
        replace, drop = {}, set()
        for i, ln in enumerate(self.ops):
            if ln['kind'] != 'layer_norm' or not ln.get('pre_addend') or ln.get('addend') or ln.get('out_dtype', 'int8') != 'int8':
                continue
            for mid, other in ((ln['lhs'], ln['pre_addend']), (ln['pre_addend'], ln['lhs'])):
                j = produced_at.get(mid)
                if j is None or j in drop or j >= i:
                    continue
                d = self.ops[j]
                if (d['kind'] != 'dense' or d['transpose_lhs'] or d['lhs_dtype'] not in ('int8', 'uint8')
                        or d.get('rhs_dtype', 'int8') != 'int8' or d['out_dtype'] != 'int8' or d['rounding'] != ln['rounding']
                        or d['N'] != ln['cols']):
                    continue
                if len(graph.tensors[mid].consumers) != 1 or mid in graph.output_tensor_names or mid in aliased:
                    continue
                if self.fmt[other] != 'int8' or self.fmt[ln['out']] != 'int8':
                    continue
                try:
                    _, M, K, lda = collapse_2d(self._view(d['lhs']), d['name'])
                    _, Mr, Nr, ldr = collapse_2d(self._view(other), ln['name'])
                    _, Mo, No, ldo = collapse_2d(self._view(ln['out']), ln['name'])
                except NotImplementedError:
                    continue
                if (M, d['N']) != (Mr, Nr) or (Mr, Nr) != (Mo, No) or K != d['K']:
                    continue
                ldw = int(self.params_np[d['weight']].shape[1])
                gmax = int(np.abs(self.params_np[ln['gamma']].astype(np.int64)).max())
                if self.lib.a4c_dense_add_layernorm_supported(M, K, d['N'], lda, ldw, ldr, ldo, d['shift'],
                                                              ROUNDING_CODE[d['rounding']], ln['out_shift'], ln['eps_q0'],
                                                              gmax) != 0:
                    continue
                name = f"{d['name']}+{ln['name']}"
                replace[i] = {'kind': 'dense_add_ln', 'name': name, 'lhs': d['lhs'], 'residual': other, 'out': ln['out'],
                              'dense': d, 'ln': ln, 'gamma_absmax': gmax}
                drop.add(j)
                self.fused.append(name)
                break
        if replace:
            self.ops = [replace.get(i, op) for i, op in enumerate(self.ops) if i not in drop]

    def _attention_args(self, op: Dict[str, Any]) -> tuple:
        """Positional arguments of a4c_attention_heads_i8 up to (not including) `rounding`, from the four views (of the
        first head when the op covers several)."""
        name = op['name']
        q, k, v, o = (self._view(op[key]) for key in ('q', 'k', 'v', 'out'))
        q_off, bq, sq, dq, ldq, stq = collapse_batched(q, f'{name}: q')
        k_off, bk, sk, dk, ldk, stk = collapse_batched(k, f'{name}: k')
        v_off, bv, sv, dv, ldv, stv = collapse_batched(v, f'{name}: v')
        o_off, bo, so, do, ldo, sto = collapse_batched(o, f'{name}: output')
        if not (bq == bk == bv == bo and sk == sv and sq == so and dq == dk == dv == do):
            raise ValueError(f'{name}: q/k/v/output shapes do not form an attention head.')
        hq, hk, hv, ho = op.get('head_strides', (0, 0, 0, 0))
        return (self.ptr(q, q_off), ldq, stq, hq, self.ptr(k, k_off), ldk, stk, hk, self.ptr(v, v_off), ldv, stv, hv,
                self.ptr(o, o_off), ldo, sto, ho, bq, op.get('heads', 1), sq, sk, dq, op['qk_shift'], op['pv_shift'])

    def _fuse_attention(self) -> None:
        """matmul(q, k^T) -> softmax (uint8) -> matmul(p, v) becomes one launch per head when the library has a
        fused kernel for the shapes (a4c_attention_i8_supported): scores and probabilities then have no
        buffer at all.  Both intermediates must feed nothing else and be neither graph outputs nor views."""
        graph = self.graph
        produced_at = {op['out']: i for i, op in enumerate(self.ops)}
        aliased = set(self.alias) | {p for p, _, _ in self.alias.values()}

        def private(t: str) -> bool:
            return len(graph.tensors[t].consumers) == 1 and t not in graph.output_tensor_names and t not in aliased

        drop, replace = set(), {}
        for i, av in enumerate(self.ops):
            if av['kind'] != 'matmul' or av['transpose_lhs'] or av['transpose_rhs'] or av['out_dtype'] != 'int8':
                continue
            j = produced_at.get(av['lhs'])
            if j is None or self.ops[j]['kind'] != 'softmax':
                continue
            sm = self.ops[j]
            if sm.get('addend') or sm['out_dtype'] != 'uint8' or not private(sm['out']) or not private(sm['lhs']):
                continue
            h = produced_at.get(sm['lhs'])
            if h is None or self.ops[h]['kind'] != 'matmul':
                continue
            qk = self.ops[h]
            if (qk['transpose_lhs'] or not qk['transpose_rhs'] or qk['out_dtype'] != 'int8' or qk['lhs_dtype'] != 'int8'
                    or qk['rounding'] != av['rounding']):
                continue
            op = {'kind': 'attention', 'name': f"{qk['name']}+{sm['name']}+{av['name']}", 'q': qk['lhs'], 'k': qk['rhs'],
                  'v': av['rhs'], 'out': av['out'], 'qk_shift': qk['shift'], 'pv_shift': av['shift'],
                  'rounding': av['rounding'], 'sm_mode': 0 if sm['approximation'] == 'hccs' else 1, 'B': sm['B'],
                  'S': sm['S'], 'Dmax': sm['Dmax'], 'inv_shift': sm['inv_shift'], 'use_clb': int(sm['use_clb']),
                  'exp_kq': sm['exp_kq']}
            if any(self.fmt[op[key]] != 'int8' for key in ('q', 'k', 'v', 'out')):
                continue
            try:
                args = self._attention_args(op)
            except (NotImplementedError, ValueError):
                continue
            if self.lib.a4c_attention_heads_i8_supported(*args, op['sm_mode'], op['B'], op['S'], op['Dmax'],
                                                   op['inv_shift']) != 0:
                continue
            replace[i] = op
            drop.update((h, j))
            self.fused.append(op['name'])
        if replace:
            self.ops = [replace.get(i, op) for i, op in enumerate(self.ops) if i not in drop]

    def _merge_attention_heads(self) -> None:
        """Fused attention ops that differ only in which column slice of the same four buffers they touch (the heads of
        one layer) become one launch over (batch entry, head): a memory line that holds several heads is then fetched
        once.  The merged op runs where the last head ran; nothing in between may touch the output buffer."""
        same = ('qk_shift', 'pv_shift', 'rounding', 'sm_mode', 'B', 'S', 'Dmax', 'inv_shift', 'use_clb', 'exp_kq')
        groups: Dict[tuple, List[int]] = {}
        for i, op in enumerate(self.ops):
            if op['kind'] != 'attention':
                continue
            vs = [self._view(op[key]) for key in ('q', 'k', 'v', 'out')]
            key = tuple(op[k] for k in same) + tuple((v.root, v.shape, v.strides) for v in vs)
            groups.setdefault(key, []).append(i)
        drop, replace = set(), {}
        for members in groups.values():
            if len(members) < 2:
                continue
            offs = {i: [self._view(self.ops[i][key]).offset for key in ('q', 'k', 'v', 'out')] for i in members}
            order = sorted(members, key=lambda i: offs[i][0])
            first = offs[order[0]]
            steps = [b - a for a, b in zip(first, offs[order[1]])]
            if any(st <= 0 for st in steps):
                continue
            if any(offs[i][c] != first[c] + h * steps[c] for h, i in enumerate(order) for c in range(4)):
                continue
            out_root = self._view(self.ops[order[0]]['out']).root
            lo, hi = min(members), max(members)
            between = [self.ops[j] for j in range(lo, hi + 1) if j not in members]
            if any(self._view(op[key]).root == out_root for op in between
                   for key in ('lhs', 'rhs', 'out', 'addend', 'pre_addend', 'q', 'k', 'v') if op.get(key)):
                continue
            head0 = self.ops[order[0]]
            merged = dict(head0, name='|'.join(self.ops[i]['name'] for i in order), heads=len(order), head_strides=tuple(steps),
                          members=[{key: self.ops[i][key] for key in ('q', 'k', 'v', 'out')} for i in order])
            try:
                args = self._attention_args(merged)
            except (NotImplementedError, ValueError):
                continue
            if self.lib.a4c_attention_heads_i8_supported(*args, merged['sm_mode'], merged['B'], merged['S'], merged['Dmax'],
                                                         merged['inv_shift']) != 0:
                continue
            replace[hi] = merged
            drop.update(i for i in members if i != hi)
            singles = {self.ops[i]['name'] for i in members}
            self.fused = [f for f in self.fused if f not in singles] + [merged['name']]
        if replace:
            self.ops = [replace.get(i, op) for i, op in enumerate(self.ops) if i not in drop]

    # ---- launch compilation --------------------------------------------------------------------
    def _compile(self, op: Dict[str, Any]) -> Tuple[Callable, tuple]:
        kind, name = op['kind'], op['name']
        L = self.lib
        if kind == 'dense':
            a, y = self._view(op['lhs']), self._view(op['out'])
            if op['transpose_lhs']:
                # the stored input is a stack of [K, M] matrices; the output a stack of [M, N]
                a_off, ba, Ks, Ms, lda, sa = collapse_batched(a, f'{name}: input')
                y_off, by, My, N, ldy, sy = collapse_batched(y, f'{name}: output')
                if (ba, Ms, Ks, N) != (by, My, op['K'], op['N']):
                    raise ValueError(f'{name}: shape mismatch between views (input {a.shape}, output {y.shape}).')
                w = self.params[op['weight']]
                bias = self.params[op['bias']] if op['bias'] else None
                args = (self.ptr(a, a_off), DTYPE_CODE[op['lhs_dtype']], lda, sa, w.data_ptr(), DTYPE_CODE[op['rhs_dtype']],
                        int(w.shape[1]), bias.data_ptr() if bias is not None else None, self.ptr(y, y_off), ldy, sy, ba,
                        Ms, Ks, N, op['shift'], ROUNDING_CODE[op['rounding']], int(op['relu']),
                        DTYPE_CODE[op['out_dtype']])
                return L.a4c_dense_ta, args
            a_off, M, K, lda = collapse_2d(a, f'{name}: input')
            y_off, My, N, ldy = collapse_2d(y, f'{name}: output')
            if (M, K, N) != (My, op['K'], op['N']):
                raise ValueError(f'{name}: shape mismatch between views (M={M}/{My}, K={K}/{op["K"]}, N={N}/{op["N"]}).')
            w = self.params[op['weight']]
            bias = self.params[op['bias']] if op['bias'] else None
            if op['lhs_dtype'] == 'int16':
                # 16-bit activations: int16 x int8 (32-bit accumulator) or int16 x int16 (64-bit accumulator)
                args = (self.ptr(a, a_off), lda, w.data_ptr(), DTYPE_CODE[op['rhs_dtype']], int(w.shape[1]),
                        bias.data_ptr() if bias is not None else None, self.ptr(y, y_off), ldy, M, K, N, op['shift'],
                        ROUNDING_CODE[op['rounding']], int(op['relu']), DTYPE_CODE[op['out_dtype']])
                return L.a4c_dense_i16, args
            args = (self.ptr(a, a_off), lda, w.data_ptr(), int(w.shape[1]), bias.data_ptr() if bias is not None else None,
                    self.ptr(y, y_off), ldy, M, K, N, op['shift'], ROUNDING_CODE[op['rounding']], int(op['relu']),
                    DTYPE_CODE[op['out_dtype']], int(op['lhs_dtype'] == 'uint8'), self.dense_algo)
            return L.a4c_dense_i8, args
        if kind == 'matmul':
            a, b, c = self._view(op['lhs']), self._view(op['rhs']), self._view(op['out'])
            a_off, ba, ar, ac, lda, sa = collapse_batched(a, f'{name}: lhs')
            b_off, bb, br, bc, ldb, sb = collapse_batched(b, f'{name}: rhs')
            c_off, bc_, M, N, ldc, sc = collapse_batched(c, f'{name}: output')
            Ka = ar if op['transpose_lhs'] else ac
            Ma = ac if op['transpose_lhs'] else ar
            Kb = bc if op['transpose_rhs'] else br
            Nb = br if op['transpose_rhs'] else bc
            if Ma != M or Nb != N or Ka != Kb:
                raise ValueError(f'{name}: operand shapes do not contract (A {a.shape}, B {b.shape}, C {c.shape}).')
            if ba != bc_ or bb not in (1, bc_):
                raise ValueError(f'{name}: batch extents differ (A {ba}, B {bb}, C {bc_}).')
            if bb == 1:
                sb = 0
            if op['lhs_dtype'] == 'int16':
                args = (self.ptr(a, a_off), lda, sa, self.ptr(b, b_off), DTYPE_CODE[op['rhs_dtype']], ldb, sb,
                        self.ptr(c, c_off), ldc, sc, bc_, M, Ka, N, int(op['transpose_lhs']), int(op['transpose_rhs']),
                        op['shift'], ROUNDING_CODE[op['rounding']], DTYPE_CODE[op['out_dtype']])
                return L.a4c_bmm_i16, args
            args = (self.ptr(a, a_off), lda, sa, self.ptr(b, b_off), ldb, sb, self.ptr(c, c_off), ldc, sc, bc_, M, Ka, N,
                    int(op['transpose_lhs']), int(op['transpose_rhs']), op['shift'], ROUNDING_CODE[op['rounding']],
                    DTYPE_CODE[op['out_dtype']], int(op['lhs_dtype'] == 'uint8'))
            return L.a4c_bmm_i8, args
        if kind == 'dense_f':
            a, y = self._view(op['lhs']), self._view(op['out'])
            a_off, M, K, lda = collapse_2d(a, f'{name}: input')
            y_off, My, N, ldy = collapse_2d(y, f'{name}: output')
            if (M, K, N) != (My, op['K'], op['N']):
                raise ValueError(f'{name}: shape mismatch between views (M={M}/{My}, K={K}/{op["K"]}, N={N}/{op["N"]}).')
            w = self.params[op['weight']]
            bias = self.params[op['bias']] if op['bias'] else None
            args = (self.ptr(a, a_off), FLOAT_CODE[op['dtype']], lda, w.data_ptr(), int(w.shape[1]),
                    bias.data_ptr() if bias is not None else None, self.ptr(y, y_off), ldy, M, K, N, int(op['relu']))
            return L.a4c_dense_f, args
        if kind == 'matmul_f':
            a, b, c = self._view(op['lhs']), self._view(op['rhs']), self._view(op['out'])
            a_off, ba, ar, ac, lda, sa = collapse_batched(a, f'{name}: lhs')
            b_off, bb, br, bc, ldb, sb = collapse_batched(b, f'{name}: rhs')
            c_off, bc_, M, N, ldc, sc = collapse_batched(c, f'{name}: output')
            Ka = ar if op['transpose_lhs'] else ac
            Ma = ac if op['transpose_lhs'] else ar
            Kb = bc if op['transpose_rhs'] else br
            Nb = br if op['transpose_rhs'] else bc
            if Ma != M or Nb != N or Ka != Kb or ba != bc_ or bb not in (1, bc_):
                raise ValueError(f'{name}: operand shapes do not contract (A {a.shape}, B {b.shape}, C {c.shape}).')
            args = (self.ptr(a, a_off), FLOAT_CODE[op['dtype']], lda, sa, self.ptr(b, b_off), ldb, 0 if bb == 1 else sb,
                    self.ptr(c, c_off), ldc, sc, bc_, M, Ka, N, int(op['transpose_lhs']), int(op['transpose_rhs']))
            return L.a4c_bmm_f, args
        if kind == 'add_f':
            x, o, y = self._view(op['lhs']), self._view(op['rhs']), self._view(op['out'])
            x_off, rows, cols, ldx = collapse_2d(x, f'{name}: lhs')
            o_off, ro, co, ldo_ = collapse_2d(o, f'{name}: rhs')
            y_off, ry, cy, ldy = collapse_2d(y, f'{name}: output')
            if (rows, cols) != (ro, co) or (rows, cols) != (ry, cy):
                raise ValueError(f'{name}: operand shapes differ.')
            args = (self.ptr(x, x_off), ldx, self.ptr(o, o_off), ldo_, self.ptr(y, y_off), ldy, rows, cols,
                    FLOAT_CODE[op['dtype']])
            return L.a4c_add_f, args
        if kind == 'mlp':
            import ctypes

            layers, dims = op['layers'], op['dims']
            a, y = self._view(op['lhs']), self._view(op['out'])
            a_off, M, K, lda = collapse_2d(a, f'{name}: input')
            y_off, My, N, ldy = collapse_2d(y, f'{name}: output')
            if M != My or K != dims[0] or N != dims[-1]:
                raise ValueError(f'{name}: chain input / output views do not match the layer sizes.')
            n = len(layers)
            ws = [self.params[l['weight']] for l in layers]
            bs = [self.params[l['bias']] if l['bias'] else None for l in layers]
            c_dims = (ctypes.c_int * (n + 1))(*dims)
            c_w = (ctypes.c_void_p * n)(*[w.data_ptr() for w in ws])
            c_ldw = (ctypes.c_int64 * n)(*[int(w.shape[1]) for w in ws])
            c_b = (ctypes.c_void_p * n)(*[b.data_ptr() if b is not None else None for b in bs])
            c_shift = (ctypes.c_int * n)(*[l['shift'] for l in layers])
            c_relu = (ctypes.c_int * n)(*[int(l['relu']) for l in layers])
            self._keepalive.append((c_dims, c_w, c_ldw, c_b, c_shift, c_relu))
            args = (self.ptr(a, a_off), lda, int(layers[0]['lhs_dtype'] == 'uint8'), n, c_dims, c_w, c_ldw, c_b, c_shift,
                    c_relu, ROUNDING_CODE[op['rounding']], self.ptr(y, y_off), ldy, DTYPE_CODE[layers[-1]['out_dtype']], M)
            return L.a4c_mlp_i8, args
        if kind == 'dense_add_ln':
            d, ln = op['dense'], op['ln']
            a, r, y = self._view(op['lhs']), self._view(op['residual']), self._view(op['out'])
            a_off, M, K, lda = collapse_2d(a, f'{name}: input')
            r_off, Mr, Nr, ldr = collapse_2d(r, f'{name}: residual')
            y_off, My, N, ldy = collapse_2d(y, f'{name}: output')
            if (M, K, N) != (My, d['K'], d['N']) or (Mr, Nr) != (M, N):
                raise ValueError(f'{name}: shape mismatch between views.')
            w = self.params[d['weight']]
            bias = self.params[d['bias']] if d['bias'] else None
            args = (self.ptr(a, a_off), lda, int(d['lhs_dtype'] == 'uint8'), w.data_ptr(), int(w.shape[1]),
                    bias.data_ptr() if bias is not None else None, d['shift'], int(d['relu']), self.ptr(r, r_off), ldr,
                    self.params[ln['gamma']].data_ptr(), self.params[ln['beta']].data_ptr(), self.ptr(y, y_off), ldy, M, K, N,
                    ln['eps_q0'], ln['out_shift'], ROUNDING_CODE[ln['rounding']], op['gamma_absmax'])
            return L.a4c_dense_add_layernorm_i8, args
        if kind == 'attention':
            args = self._attention_args(op) + (ROUNDING_CODE[op['rounding']], op['sm_mode'], op['B'], op['S'],
                                               op['Dmax'], op['inv_shift'], op['use_clb'], op['exp_kq'])
            return L.a4c_attention_heads_i8, args
        if kind in ('layer_norm', 'softmax', 'add'):
            x, y = self._view(op['lhs']), self._view(op['out'])
            x_off, rows, cols, ldx = collapse_2d(x, f'{name}: input')
            y_off, rows_y, cols_y, ldy = collapse_2d(y, f'{name}: output')
            if (rows, cols) != (rows_y, cols_y):
                raise ValueError(f'{name}: input and output views differ in shape.')
            add_ptr, ldadd = None, 0
            other = (op.get('addend') or op.get('pre_addend')) if kind != 'add' else op['rhs']
            if other:
                o = self._view(other)
                o_off, ro, co, ldadd = collapse_2d(o, f'{name}: addend')
                if (ro, co) != (rows, cols):
                    raise ValueError(f'{name}: addend shape differs from the output.')
                add_ptr = self.ptr(o, o_off)
            if kind == 'layer_norm' and op.get('pre_addend'):
                args = (self.ptr(x, x_off), ldx, add_ptr, ldadd, self.params[op['gamma']].data_ptr(),
                        self.params[op['beta']].data_ptr(), self.ptr(y, y_off), ldy, rows, cols, op['eps_q0'],
                        op['out_shift'], ROUNDING_CODE[op['rounding']],
                        int(np.abs(self.params_np[op['gamma']].astype(np.int64)).max()))
                return L.a4c_add_layernorm_i8, args
            if kind == 'layer_norm':
                args = (self.ptr(x, x_off), ldx, self.params[op['gamma']].data_ptr(), self.params[op['beta']].data_ptr(),
                        add_ptr, ldadd, self.ptr(y, y_off), ldy, rows, cols, op['eps_q0'], op['out_shift'],
                        ROUNDING_CODE[op['rounding']], int(np.abs(self.params_np[op['gamma']].astype(np.int64)).max()))
                return L.a4c_layernorm_i8, args
            if kind == 'softmax':
                args = (self.ptr(x, x_off), ldx, add_ptr, ldadd, self.ptr(y, y_off), ldy, rows, cols,
                        0 if op['approximation'] == 'hccs' else 1, op['B'], op['S'], op['Dmax'], op['inv_shift'],
                        int(op['use_clb']), op['exp_kq'], DTYPE_CODE[op['out_dtype']])
                return L.a4c_softmax_i8, args
            args = (self.ptr(x, x_off), ldx, add_ptr, ldadd, self.ptr(y, y_off), ldy, rows, cols, op['shift'],
                    ROUNDING_CODE[op['rounding']], DTYPE_CODE[op['out_dtype']])
            return L.a4c_add_sat, args
        raise NotImplementedError(f'{name}: no launch rule for op kind {kind!r}.')

    # ---- execution -----------------------------------------------------------------------------
    def launch_all(self, stream_handle: int) -> None:
        for (fn, args), op in zip(self.launches, self.ops):
            rc = fn(*args, stream_handle)
            if rc != 0:
                _lib.check(rc, f"{op['name']} ({op['kind']})")

    def run(self, use_graph: bool = True) -> None:
        """Execute every launch on the current stream (replaying a captured CUDA graph once one exists)."""
        torch = _torch()
        with torch.cuda.device(self.device):
            if use_graph and self.graph_exec is not None:
                self.graph_exec.replay()
                return
            self.launch_all(torch.cuda.current_stream(self.device).cuda_stream)

    def capture(self) -> None:
        """Capture the launch list into a CUDA graph (after one eager warm-up run)."""
        torch = _torch()
        with torch.cuda.device(self.device):
            self.run(use_graph=False)
            torch.cuda.synchronize(self.device)
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                self.launch_all(torch.cuda.current_stream(self.device).cuda_stream)
            self.graph_exec = g

    def check_status(self) -> None:
        torch = _torch()
        with torch.cuda.device(self.device):
            _lib.device_status(torch.cuda.current_stream(self.device).cuda_stream)

    # ---- export --------------------------------------------------------------------------------
    def export(self) -> Dict[str, Any]:
        """The lowered plan as plain data: what the CPU oracle evaluates and what a dump records."""
        ops: List[Dict[str, Any]] = []
        params: Dict[str, np.ndarray] = {}
        for node in self.graph.nodes:
            if node.is_placeholder:
                if 'slice_view' in node.traits:
                    d = node.traits['slice_view'].data
                    ops.append({'kind': 'slice', 'name': node.name, 'source': d['source'], 'axis': d['axis'],
                                'slices': [dict(s) for s in d['slices']]})
                else:
                    d = node.traits['concat_view'].data
                    ops.append({'kind': 'concat', 'name': node.name, 'out': d['output'], 'axis': d['axis'],
                                'inputs': [s['input'] for s in d['slices']]})
                continue
            inst = self.ctx.ir.execution.get(node.name)
            op = inst.variant.plan_op(inst)
            if op['kind'] in ('dense', 'dense_f'):
                params[op['weight']] = inst.artifacts['weights_kn']
                if op['bias']:
                    params[op['bias']] = inst.artifacts['packed_bias']
            elif op['kind'] == 'layer_norm':
                params[op['gamma']] = inst.artifacts['packed_gamma']
                params[op['beta']] = inst.artifacts['packed_beta']
            ops.append(op)
        return {'inputs': list(self.graph.input_tensor_names), 'outputs': list(self.graph.output_tensor_names),
                'ops': ops, 'params': params, 'fused': list(self.fused),
                'formats': dict(self.fmt)}
