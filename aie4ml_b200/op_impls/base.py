"""The operator-implementation boundary of the CUDA target.

Mirrors the reference's plugin interface (``src/aie4ml/op_impls/base.py:19-88``,
``registry.py:11-47``, ``family_registry.py:9-57``): one ``OpImplVariant`` per kernel flavour,
registered under its ``op_type``; a ``FamilyResolver`` per op type validates structure and picks
the highest-``plevel`` variant whose ``matches`` accepts the node.  The AIE-only half of that
interface (ports, staging descriptors, footprints, Jinja parameter templates) has no GPU meaning
and is not part of this boundary.
"""

from __future__ import annotations

from typing import Any, ClassVar, Dict, List, Optional, Tuple

from ..ir import ExecutionEntry, OpNode

CUDA_GENERATIONS = ('CUDA-SM100',)


class OpImplVariant:
    variant_id: ClassVar[str] = ''
    op_type: ClassVar[str] = ''
    plevel: ClassVar[int] = 10  # higher = tried first

    def matches(self, _node: OpNode, _device: Any) -> bool:
        raise NotImplementedError

    def resolve(self, _node: OpNode, _device: Any, _directives: Optional[Dict[str, Any]] = None) -> Any:
        raise NotImplementedError

    def validate_config(self, _node: OpNode, _config: Any, _device: Any) -> None:
        """Post-resolution verifier; raise ValueError naming the node."""

    def pack(self, inst: ExecutionEntry) -> Dict[str, Any]:
        return {}

    def get_artifacts(self, inst: ExecutionEntry) -> List[Dict[str, Any]]:
        return []

    def input_precision(self, config: Any, role: str) -> Any:
        return config.precision[role]

    def output_precision(self, config: Any) -> Any:
        return config.precision['output']

    def plan_op(self, inst: ExecutionEntry) -> Dict[str, Any]:
        """Describe this node as a plain dict for the runtime / plan export."""
        raise NotImplementedError


class OpImplRegistry:
    def __init__(self) -> None:
        self._variants: Dict[str, List[OpImplVariant]] = {}

    def register(self, variant: OpImplVariant) -> None:
        self._variants.setdefault(variant.op_type, []).append(variant)

    def candidates(self, op_type: str) -> List[OpImplVariant]:
        return sorted(self._variants.get(op_type, []), key=lambda v: -v.plevel)


_REGISTRY = OpImplRegistry()


def get_op_impl_registry() -> OpImplRegistry:
    return _REGISTRY


def register_variant(cls):
    _REGISTRY.register(cls())
    return cls


class FamilyResolver:
    op_type: ClassVar[str] = ''

    def validate_structure(self, _node: Any, _device: Any) -> None:
        raise NotImplementedError

    def resolve(self, node: Any, device: Any, directives: Optional[Dict[str, Any]] = None) -> Tuple[Any, OpImplVariant]:
        self.validate_structure(node, device)
        for variant in _REGISTRY.candidates(self.op_type):
            if variant.matches(node, device):
                return variant.resolve(node, device, directives), variant
        raise ValueError(f'{node.name}: no {self.op_type} variant matches (generation={device.generation!r}).')


class FamilyResolverRegistry:
    def __init__(self) -> None:
        self._resolvers: Dict[str, FamilyResolver] = {}

    def register(self, op_type: str, resolver: FamilyResolver) -> None:
        self._resolvers[op_type] = resolver

    def get(self, op_type: str) -> FamilyResolver:
        try:
            return self._resolvers[op_type]
        except KeyError:
            raise NotImplementedError(f'No family resolver registered for op_type={op_type!r}.') from None


_FAMILIES = FamilyResolverRegistry()


def get_family_resolver_registry() -> FamilyResolverRegistry:
    return _FAMILIES


def family_resolver(*op_types: str):
    def decorate(cls):
        inst = cls()
        for op_type in op_types:
            _FAMILIES.register(str(op_type), inst)
        return cls

    return decorate
