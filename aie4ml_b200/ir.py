"""Logical and execution IR of the lowered, quantized operator graph.

The class and field names follow the reference's ``src/aie4ml/ir/graph.py`` (TensorVar :17-34,
OpNode :52-75, LogicalIR :103-276, ExecutionEntry :311-333, ExecutionIR :339-393) so that
frontends and passes written against the reference read the same here.  The AIE-physical
third level (placement, memory-tile plan) has no counterpart on a GPU and is absent.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, Iterable, List, Optional, Sequence, Tuple

import numpy as np


@dataclass
class TensorVar:
    """A logical tensor.  Parameters carry ``data`` (float values, not yet quantised) and have
    no producer; activations have a producer node (or are graph inputs)."""

    name: str
    shape: Tuple[int, ...]
    precision: Optional[Any] = None
    data: Optional[np.ndarray] = None
    producer: Optional['OpNode'] = None
    consumers: List['OpNode'] = field(default_factory=list)

    @property
    def is_parameter(self) -> bool:
        return self.data is not None


@dataclass
class TraitInstance:
    name: str
    data: Dict[str, Any] = field(default_factory=dict)


@dataclass
class OpNode:
    name: str
    op_type: str
    dialect: str = 'cuda'
    inputs: List[TensorVar] = field(default_factory=list)
    outputs: List[TensorVar] = field(default_factory=list)
    artifacts: Dict[str, Any] = field(default_factory=dict)
    traits: Dict[str, TraitInstance] = field(default_factory=dict)
    metadata: Dict[str, Any] = field(default_factory=dict)
    directives: Dict[str, Any] = field(default_factory=dict)
    roles: Dict[str, str] = field(default_factory=dict)
    is_placeholder: bool = False

    def add_trait(self, trait: TraitInstance) -> None:
        self.traits[trait.name] = trait

    def trait_data(self, name: str) -> Dict[str, Any]:
        trait = self.traits.get(name)
        return trait.data if trait is not None else {}

    def __hash__(self) -> int:  # identity hash: nodes are graph vertices
        return id(self)

    def __eq__(self, other) -> bool:
        return self is other


def set_input_roles(node: OpNode, tensors: Sequence[TensorVar], role_names: Sequence[str]) -> None:
    if len(tensors) != len(role_names):
        raise ValueError(f'{node.name}: set_input_roles got {len(tensors)} tensors but {len(role_names)} role names.')
    node.roles = {t.name: str(r) for t, r in zip(tensors, role_names)}


def input_role(node: OpNode, tensor_name: str) -> Optional[str]:
    return node.roles.get(tensor_name)


def input_tensor_for_role(node: OpNode, role: str) -> TensorVar:
    for tensor in node.inputs:
        if node.roles.get(tensor.name) == role:
            return tensor
    raise ValueError(f'{node.name}: missing {role} tensor.')


def optional_tensor_for_role(node: OpNode, role: str) -> Optional[TensorVar]:
    for tensor in node.inputs:
        if node.roles.get(tensor.name) == role:
            return tensor
    return None


@dataclass
class LogicalIR:
    """Tensor-centric graph: tensors by name, nodes in topological order."""

    tensors: Dict[str, TensorVar] = field(default_factory=dict)
    nodes: List[OpNode] = field(default_factory=list)
    input_tensor_names: List[str] = field(default_factory=list)
    output_tensor_names: List[str] = field(default_factory=list)

    def add_tensor(self, tensor: TensorVar) -> None:
        if tensor.name in self.tensors:
            raise ValueError(f"Tensor '{tensor.name}' already exists.")
        self.tensors[tensor.name] = tensor

    def add_node(self, node: OpNode) -> None:
        self.nodes.append(node)

    def mark_graph_input(self, tensor_name: str) -> None:
        if tensor_name not in self.tensors:
            raise ValueError(f"Graph input tensor '{tensor_name}' does not exist.")
        if tensor_name not in self.input_tensor_names:
            self.input_tensor_names.append(tensor_name)

    def mark_graph_output(self, tensor_name: str) -> None:
        if tensor_name not in self.tensors:
            raise ValueError(f"Graph output tensor '{tensor_name}' does not exist.")
        if tensor_name not in self.output_tensor_names:
            self.output_tensor_names.append(tensor_name)

    def graph_inputs(self) -> List[TensorVar]:
        return [self.tensors[n] for n in self.input_tensor_names]

    def graph_outputs(self) -> List[TensorVar]:
        return [self.tensors[n] for n in self.output_tensor_names]

    # -- node removal ----------------------------------------------------------------------
    def remove_node(self, node: OpNode, mode: str = 'bypass') -> None:
        """Remove a 1-in/1-out node.

        ``bypass``: consumers of the output read the node's input instead (output tensor dies).
        ``contract``: the producer of the input writes the node's output instead (input tensor
        dies); only legal when the input has no other consumer.
        """
        if len(node.inputs) != 1 or len(node.outputs) != 1:
            raise ValueError(f'Cannot remove node {node.name}: expected one input and one output.')
        src, dst = node.inputs[0], node.outputs[0]
        if mode == 'bypass':
            for user in list(dst.consumers):
                user.inputs = [src if t is dst else t for t in user.inputs]
                if user not in src.consumers:
                    src.consumers.append(user)
                if dst.name in user.roles:
                    user.roles[src.name] = user.roles.pop(dst.name)
            src.consumers = [c for c in src.consumers if c is not node]
            if dst.name in self.output_tensor_names:
                self.output_tensor_names = [src.name if n == dst.name else n for n in self.output_tensor_names]
            self.tensors.pop(dst.name, None)
        elif mode == 'contract':
            if len(src.consumers) != 1:
                raise ValueError(
                    f'Cannot contract node {node.name}: input tensor {src.name} has {len(src.consumers)} consumers.')
            producer = src.producer
            if producer is not None:
                producer.outputs = [dst if t is src else t for t in producer.outputs]
            dst.producer = producer
            if producer is None and src.name in self.input_tensor_names:
                self.input_tensor_names = [dst.name if n == src.name else n for n in self.input_tensor_names]
            self.tensors.pop(src.name, None)
        else:
            raise ValueError(f'Unknown mode: {mode}')
        self.nodes = [n for n in self.nodes if n is not node]
        node.inputs, node.outputs = [], []

    # -- invariants ------------------------------------------------------------------------
    def verify(self) -> None:
        seen_nodes = set()
        for node in self.nodes:
            if node.name in seen_nodes:
                raise RuntimeError(f'LogicalIR has duplicate node name {node.name!r}.')
            for tensor in node.inputs:
                if tensor.is_parameter:
                    continue
                if tensor.producer is None:
                    if tensor.name not in self.input_tensor_names:
                        raise RuntimeError(f'{node.name}: activation input {tensor.name!r} has no producer and is '
                                           'not a declared graph input.')
                elif tensor.producer.name not in seen_nodes:
                    raise RuntimeError(f'LogicalIR is not in topological order: {node.name!r} consumes '
                                       f'{tensor.name!r} before its producer {tensor.producer.name!r}.')
            seen_nodes.add(node.name)

    def __iter__(self):
        return iter(self.nodes)

    def __len__(self) -> int:
        return len(self.nodes)


@dataclass
class ExecutionEntry:
    """The implementation selected for one logical node plus its resolved numeric contract."""

    node: OpNode
    variant: Any
    config: Any
    artifacts: Dict[str, Any] = field(default_factory=dict)

    @property
    def name(self) -> str:
        return self.node.name

    @property
    def op_type(self) -> str:
        return self.node.op_type


OpImplInstance = ExecutionEntry


@dataclass
class ExecutionIR:
    instances: Dict[str, ExecutionEntry] = field(default_factory=dict)

    def register(self, node: OpNode, variant: Any, config: Any) -> ExecutionEntry:
        inst = ExecutionEntry(node=node, variant=variant, config=config)
        self.instances[node.name] = inst
        return inst

    def get(self, name: str) -> Optional[ExecutionEntry]:
        return self.instances.get(name)

    def prune(self, active: Iterable[str]) -> bool:
        keep = set(active)
        dead = [n for n in self.instances if n not in keep]
        for n in dead:
            del self.instances[n]
        return bool(dead)

    def __iter__(self):
        return iter(self.instances.values())


@dataclass
class PipelineIR:
    logical: LogicalIR = field(default_factory=LogicalIR)
    execution: ExecutionIR = field(default_factory=ExecutionIR)


@dataclass(frozen=True)
class DeviceSpec:
    """Execution target.  ``generation`` plays the role the reference's AIE generation string
    plays in every variant's ``matches`` (e.g. op_impls/families/softmax/softmax.py:67-78)."""

    part: str = 'cuda_b200'
    generation: str = 'CUDA-SM100'
    dialect: str = 'cuda'
    sm_count: int = 148
    hbm_bytes: int = 180 * (1 << 30)


DEVICE_CATALOG = {
    'cuda_b200': DeviceSpec(),
}


@dataclass
class BackendContext:
    device: DeviceSpec = field(default_factory=DeviceSpec)
    aie_config: Dict[str, Any] = field(default_factory=dict)
    project_name: str = 'model'
    output_dir: Optional[str] = None
    ir: PipelineIR = field(default_factory=PipelineIR)


def get_backend_context(model_or_ctx) -> BackendContext:
    if isinstance(model_or_ctx, BackendContext):
        return model_or_ctx
    ctx = getattr(model_or_ctx, 'context', None)
    if isinstance(ctx, BackendContext):
        return ctx
    raise TypeError('expected a BackendContext or an object exposing .context')
