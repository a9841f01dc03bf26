"""Semantic lowering passes run between a frontend's logical IR and the CUDA runtime.

Same pass names, order and effects as the hardware-agnostic head of the reference pipeline
(``src/aie4ml/pipeline.py:21-39``): FoldBias (``passes/fold_bias.py:12-81``), FoldScale
(``passes/fold_scale.py:10-72``), FuseActivationCasts (``passes/fuse_activation.py:7-41``),
FoldViewOps (``passes/fold_views.py:7-150``), Resolve (``passes/resolve.py:41-95``) and
PackKernelArtifacts (``passes/pack.py:11-37``).  The AIE-physical tail of that pipeline
(transport, placement, memory-tile planning) is replaced by the runtime's buffer/view plan.
"""

from __future__ import annotations

from typing import Iterable

import numpy as np

from .ir import BackendContext, OpNode, TraitInstance, get_backend_context
from .op_impls import get_family_resolver_registry
from .op_impls.views import ensure_io_view


class AIEPass:
    name: str = ''

    def transform(self, model_or_ctx) -> bool:
        raise NotImplementedError


class FoldBias(AIEPass):
    """``add(dense_out, const)`` -> the dense's bias input (frontends emit Gemm bias as an add)."""

    name = 'fold_bias'

    def transform(self, model_or_ctx) -> bool:
        graph = get_backend_context(model_or_ctx).ir.logical
        changed = False
        for add in list(graph.nodes):
            if add.op_type != 'add' or len(add.inputs) != 2 or len(add.outputs) != 1:
                continue
            a, b = add.inputs
            if self._biasless_dense_output(a) and b.is_parameter:
                pre, bias = a, b
            elif self._biasless_dense_output(b) and a.is_parameter:
                pre, bias = b, a
            else:
                continue
            dense = pre.producer
            n_out = int(dense.metadata['n_out'])
            n_bias = int(np.asarray(bias.data).size)
            if n_bias != n_out:
                raise ValueError(f'{add.name}: dense bias Add requires exactly {n_out} elements, got {n_bias}.')
            if len(pre.consumers) != 1:
                raise ValueError(f'{add.name}: cannot fold bias because dense output {pre.name!r} '
                                 f'has {len(pre.consumers)} consumers.')
            out = add.outputs[0]
            dense.inputs.append(bias)
            bias.consumers = [c for c in bias.consumers if c is not add] + [dense]
            dense.metadata['use_bias'] = True
            dense.metadata['input_roles'] = ['lhs', 'rhs', 'bias']
            dense.roles[bias.name] = 'bias'
            dense.outputs = [out]
            out.producer = dense
            graph.tensors.pop(pre.name, None)
            graph.nodes = [n for n in graph.nodes if n is not add]
            add.inputs, add.outputs = [], []
            changed = True
        return changed

    @staticmethod
    def _biasless_dense_output(tensor) -> bool:
        p = tensor.producer
        return p is not None and p.op_type == 'dense' and not p.metadata.get('use_bias')


# which ops can swallow a constant scale, and on which side
_SCALE_ABSORBERS = {'dense': 'output_scale', 'matmul': 'output_scale', 'softmax': 'input_scale'}


class FoldScale(AIEPass):
    """Fold a scalar ``scale`` node into its consumer (softmax temperature) if that absorbs
    input scales, else into its producer (dense / matmul output shift).  Anything else is an
    error: there is no standalone scale kernel."""

    name = 'fold_scale'

    def transform(self, model_or_ctx) -> bool:
        graph = get_backend_context(model_or_ctx).ir.logical
        changed = False
        for node in list(graph.nodes):
            if node.op_type != 'scale':
                continue
            if len(node.inputs) != 1 or len(node.outputs) != 1:
                raise ValueError(f'{node.name}: scale must have exactly one input and one output.')
            scale = float(node.metadata['scale'])
            if scale <= 0.0:
                raise ValueError(f'{node.name}: scale must be positive, got {scale}.')
            src = node.inputs[0]
            users = list(node.outputs[0].consumers)
            user = users[0] if len(users) == 1 else None
            producer = src.producer
            if user is not None and _SCALE_ABSORBERS.get(user.op_type) == 'input_scale':
                self._accumulate(user, 'input_scale', scale)
                graph.remove_node(node, mode='bypass')
            elif producer is not None and _SCALE_ABSORBERS.get(producer.op_type) == 'output_scale':
                if len(src.consumers) != 1:
                    raise NotImplementedError(f'{node.name}: cannot fold output scale because {src.name!r} '
                                              f'has {len(src.consumers)} consumers.')
                self._accumulate(producer, 'output_scale', scale)
                graph.remove_node(node, mode='contract')
            else:
                raise NotImplementedError(
                    f'{node.name}: no adjacent op absorbs this scale (producer='
                    f'{producer.op_type if producer else None}, consumers={[c.op_type for c in users]}); '
                    'there is no standalone scale kernel.')
            changed = True
        return changed

    @staticmethod
    def _accumulate(node: OpNode, trait_name: str, scale: float) -> None:
        prev = node.traits.get(trait_name)
        total = scale * float(prev.data['scale']) if prev is not None else scale
        node.add_trait(TraitInstance(trait_name, {'scale': total}))


class FuseActivationCasts(AIEPass):
    """ReLU after a dense becomes the dense's ``fused_activation`` trait; linear activations are
    pure precision casts and are contracted away.  The output tensor keeps the post-activation
    precision."""

    name = 'fuse_activation_casts'

    def transform(self, model_or_ctx) -> bool:
        graph = get_backend_context(model_or_ctx).ir.logical
        changed = False
        for act in list(graph.nodes):
            if act.op_type != 'activation' or len(act.inputs) != 1 or len(act.outputs) != 1:
                continue
            kind = (act.metadata.get('activation', '') or '').lower()
            if kind == 'relu':
                producer = act.inputs[0].producer
                if producer is None or producer.op_type != 'dense' or len(producer.outputs) != 1:
                    continue
                producer.add_trait(TraitInstance('fused_activation', {'activation': 'relu'}))
                graph.remove_node(act, mode='contract')
                changed = True
            elif kind in ('linear', ''):
                graph.remove_node(act, mode='contract')
                changed = True
        return changed


class FoldViewOps(AIEPass):
    """Transpose -> ``io_view.perm`` on each consumer; Concat / Slice / Split -> placeholder nodes
    carrying ``concat_view`` / ``slice_view`` traits.  None of them ever runs a kernel."""

    name = 'fold_view_ops'

    def transform(self, model_or_ctx) -> bool:
        graph = get_backend_context(model_or_ctx).ir.logical
        changed = False
        for node in list(graph.nodes):
            if node.op_type == 'transpose':
                self._fold_transpose(graph, node)
            elif node.op_type == 'concat':
                self._fold_concat(node)
            elif node.op_type in ('slice', 'split'):
                self._fold_slice(node)
            else:
                continue
            changed = True
        return changed

    @staticmethod
    def _io_view(node: OpNode) -> dict:
        trait = node.traits.get('io_view')
        if trait is None:
            trait = TraitInstance('io_view', {'inputs': {}, 'outputs': {}})
            node.add_trait(trait)
        trait.data.setdefault('inputs', {})
        trait.data.setdefault('outputs', {})
        return trait.data

    def _fold_transpose(self, graph, node: OpNode) -> None:
        src, dst = node.inputs[0], node.outputs[0]
        perm = node.metadata.get('perm')
        if perm is None:
            raise ValueError(f'{node.name}: missing transpose permutation metadata.')
        perm = [int(p) for p in perm]
        rank = len(src.shape)
        if len(dst.shape) != rank:
            raise ValueError(f'{node.name}: transpose rank mismatch between input and output.')
        if sorted(perm) != list(range(rank)):
            raise ValueError(f'{node.name}: invalid permutation {perm} for rank {rank}.')
        if dst.name in graph.output_tensor_names:
            raise NotImplementedError(f'{node.name}: a Transpose feeding a graph output has no kernel.')
        for user in dst.consumers:
            views = self._io_view(user)['inputs']
            views[src.name] = {'perm': list(perm)}
            views.pop(dst.name, None)
        graph.remove_node(node, mode='bypass')

    @staticmethod
    def _fold_concat(node: OpNode) -> None:
        if len(node.outputs) != 1:
            raise ValueError(f'{node.name}: concat must have exactly one output.')
        if not node.inputs:
            raise ValueError(f'{node.name}: concat must have at least one input.')
        out = node.outputs[0]
        rank = len(out.shape)
        axis = int(node.metadata.get('axis', -1))
        axis = axis + rank if axis < 0 else axis
        if not 0 <= axis < rank:
            raise ValueError(f'{node.name}: concat axis {node.metadata.get("axis")} is out of range for rank {rank}.')
        cursor, pieces = 0, []
        for t in node.inputs:
            if len(t.shape) != rank:
                raise ValueError(f'{node.name}: concat input {t.name!r} rank does not match output rank.')
            pieces.append({'input': t.name, 'start': cursor, 'extent': int(t.shape[axis])})
            cursor += int(t.shape[axis])
        if cursor != int(out.shape[axis]):
            raise ValueError(f'{node.name}: concat output axis extent {out.shape[axis]} does not match input sum '
                             f'{cursor}.')
        node.add_trait(TraitInstance('concat_view', {'kind': 'concat', 'axis': axis, 'output': out.name,
                                                     'slices': pieces}))
        node.is_placeholder = True

    @staticmethod
    def _fold_slice(node: OpNode) -> None:
        if len(node.inputs) != 1:
            raise ValueError(f'{node.name}: {node.op_type} view must have exactly one input.')
        if not node.outputs:
            raise ValueError(f'{node.name}: {node.op_type} view must have at least one output.')
        src = node.inputs[0]
        rank = len(src.shape)
        axis = int(node.metadata['axis'])
        axis = axis + rank if axis < 0 else axis
        if not 0 <= axis < rank:
            raise ValueError(f'{node.name}: {node.op_type} axis {axis} is out of range for rank {rank}.')
        ranges = list(node.metadata.get('slices', ()))
        if len(ranges) != len(node.outputs):
            raise ValueError(f'{node.name}: {node.op_type} slice metadata does not match output count.')
        pieces = []
        for out, item in zip(node.outputs, ranges):
            start, extent = int(item['start']), int(item['extent'])
            if start < 0 or extent <= 0 or start + extent > int(src.shape[axis]):
                raise ValueError(f'{node.name}: invalid {node.op_type} range [{start}, {start + extent}).')
            if int(out.shape[axis]) != extent:
                raise ValueError(f'{node.name}: {node.op_type} output {out.name!r} extent mismatch.')
            pieces.append({'output': out.name, 'start': start, 'extent': extent})
        node.add_trait(TraitInstance('slice_view', {'kind': node.op_type, 'axis': axis, 'source': src.name,
                                                    'slices': pieces}))
        node.is_placeholder = True


class Resolve(AIEPass):
    """Pick an implementation variant for every non-placeholder node and freeze its numeric
    contract into an execution entry."""

    name = 'resolve'

    def transform(self, model_or_ctx) -> bool:
        ctx = get_backend_context(model_or_ctx)
        ctx.ir.logical.verify()
        registry = get_family_resolver_registry()
        visited, changed = set(), False
        for node in ctx.ir.logical:
            if node.is_placeholder:
                continue
            resolver = registry.get(node.op_type)
            ensure_io_view(node, ctx.device.generation)
            config, variant = resolver.resolve(node, ctx.device, dict(node.directives or {}))
            variant.validate_config(node, config, ctx.device)
            prev = ctx.ir.execution.get(node.name)
            if prev is None or prev.variant is not variant or prev.config != config:
                ctx.ir.execution.register(node, variant, config)
                changed = True
            visited.add(node.name)
        return ctx.ir.execution.prune(visited) or changed


class PackKernelArtifacts(AIEPass):
    """Quantise and lay out kernel-resident constants (weights, bias, gamma, beta)."""

    name = 'pack_kernel_artifacts'

    def transform(self, model_or_ctx) -> bool:
        ctx = get_backend_context(model_or_ctx)
        changed = False
        for inst in ctx.ir.execution:
            if inst.artifacts:
                continue
            packed = inst.variant.pack(inst)
            if packed:
                inst.artifacts.update(packed)
                changed = True
        return changed


class ForceFloatMode(AIEPass):
    """Replaces every quantisation intent in the logical IR by a floating-point one when ``AIEConfig.ComputeDtype``
    is ``'bfloat16'`` or ``'float32'`` / ``'float'`` (reference ``passes/force_float_mode.py:22-46``): the graph
    is then computed in that type -- Dense / MatMul with float32 accumulation, Add, ReLU -- instead of integers."""

    name = 'force_float_mode'
    _FORMATS = {'bfloat16': ('BF16', 16), 'float32': ('FP32', 32), 'float': ('FP32', 32)}

    def transform(self, ctx: BackendContext) -> bool:
        from .qtypes import FloatFormat, FloatIntent, QuantIntent

        fmt = str(ctx.aie_config.get('ComputeDtype') or '').lower()
        if not fmt:
            return False
        if fmt not in self._FORMATS:
            raise ValueError(f'ComputeDtype={fmt!r} is not recognised. Use one of: {list(self._FORMATS)}')
        name, width = self._FORMATS[fmt]
        intent = FloatIntent(width=width, format=FloatFormat[name])
        changed = False
        for t in ctx.ir.logical.tensors.values():
            if isinstance(t.precision, QuantIntent):
                t.precision = intent
                changed = True
        return changed


DEFAULT_PIPELINE = (ForceFloatMode, FoldBias, FoldScale, FuseActivationCasts, FoldViewOps, Resolve, PackKernelArtifacts)


def run_aie_passes(ctx: BackendContext, passes: Iterable[AIEPass]) -> None:
    ctx.ir.logical.verify()
    for p in passes:
        p.transform(ctx)
