"""io_view helpers: how a node sees its operands after Transpose folding.

Reference: ``src/aie4ml/op_impls/utils/io.py`` -- ensure_io_view :9-27, view_shape :89-97,
view_layout :100-104.  A folded Transpose leaves ``{'perm': [...]}`` on the consumer's
``io_view.inputs[tensor]``; an empty dict is the identity view.
"""

from __future__ import annotations

from typing import Any, Dict, List, Optional

from ..ir import TraitInstance

MAX_RANK = 5


def ensure_io_view(node, _generation: str = '') -> None:
    trait = node.traits.get('io_view')
    if trait is None:
        trait = TraitInstance('io_view', {'inputs': {}, 'outputs': {}})
        node.add_trait(trait)
    trait.data.setdefault('inputs', {})
    trait.data.setdefault('outputs', {})
    for direction, tensors in (('inputs', node.inputs), ('outputs', node.outputs)):
        for tensor in tensors:
            if len(tensor.shape) > MAX_RANK:
                raise ValueError(f'{node.name}: tensor rank {len(tensor.shape)} exceeds max {MAX_RANK}.')
            trait.data[direction].setdefault(tensor.name, {})


def view_layout(node, tensor, direction: str) -> Dict[str, Any]:
    trait = node.traits.get('io_view')
    if trait is None:
        return {}
    return trait.data.get(direction, {}).get(tensor.name, {})


def view_perm(node, tensor, direction: str = 'inputs') -> Optional[List[int]]:
    perm = view_layout(node, tensor, direction).get('perm')
    return [int(p) for p in perm] if perm is not None else None


def view_shape(node, tensor, direction: str) -> List[int]:
    logical = [int(x) for x in tensor.shape]
    perm = view_perm(node, tensor, direction)
    if perm is None:
        return logical
    if sorted(perm) != list(range(len(logical))):
        raise ValueError(f'{node.name}: invalid io_view perm {perm} for rank {len(logical)}.')
    return [logical[i] for i in perm]


def is_last_two_swap(perm: Optional[List[int]]) -> bool:
    if perm is None or len(perm) < 2:
        return False
    want = list(range(len(perm)))
    want[-1], want[-2] = want[-2], want[-1]
    return list(perm) == want


def is_identity(perm: Optional[List[int]]) -> bool:
    return perm is None or list(perm) == list(range(len(perm)))
