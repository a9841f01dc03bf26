"""Operator contracts of the CUDA target; importing this package registers every variant."""

from .base import (
    FamilyResolver,
    OpImplVariant,
    family_resolver,
    get_family_resolver_registry,
    get_op_impl_registry,
    register_variant,
)
from . import add, floatsim, layernorm, matmul, softmax  # noqa: F401  (registration side effects)

__all__ = [
    'FamilyResolver',
    'OpImplVariant',
    'family_resolver',
    'get_family_resolver_registry',
    'get_op_impl_registry',
    'register_variant',
]
