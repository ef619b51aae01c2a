"""
Applies a list of :class:`StateMappingTemplate` to a state dict
(API of src/olmo_core/nn/conversion/state_converter.py:18-146).
"""

from __future__ import annotations

import itertools
from dataclasses import dataclass
from typing import Any, Dict, List, Optional

import torch

from .state_mapping import StateMapping, StateMappingTemplate, StateType, TemplatePlaceholder

__all__ = ["StateConverter"]


@dataclass
class StateConverter:
    mapping_templates: List[StateMappingTemplate]

    def get_mappings(self, state_dict: Dict[str, Any], placeholder_bounds: Dict[TemplatePlaceholder, int],
                     state_type: StateType = StateType.weight) -> List[StateMapping]:
        """Every concrete mapping whose source keys are all present in ``state_dict`` (nothing is converted)."""
        # each placeholder takes every value below its bound, or no value at all (keys without that placeholder)
        axes = [[(p, v) for v in (*range(bound), None)] for p, bound in placeholder_bounds.items()]
        combos: List[Dict[TemplatePlaceholder, Optional[int]]] = [dict(c) for c in itertools.product(*axes)]
        present = set(state_dict)
        found: List[StateMapping] = []
        for template in self.mapping_templates:
            if template.state_type != state_type:
                continue
            for combo in combos:
                mapping = template.to_mapping(combo, placeholder_bounds)
                if mapping is not None and present.issuperset(mapping.source_keys):
                    found.append(mapping)
        return found

    def convert(self, state_dict: Dict[str, Any], placeholder_bounds: Dict[TemplatePlaceholder, int],
                state_type: StateType = StateType.weight) -> Dict[str, Any]:
        """Convert tensors; raises if a key of ``state_dict`` is covered by no mapping."""
        out: Dict[str, Any] = {}
        leftover = set(state_dict)
        for m in self.get_mappings(state_dict, placeholder_bounds, state_type):
            parts = [state_dict[k] for k in m.source_keys]
            if not all(isinstance(t, torch.Tensor) for t in parts):
                raise RuntimeError(f"only tensors can be converted ({m.source_keys} -> {m.dest_keys})")
            t = parts[0] if len(parts) == 1 else torch.cat(parts, dim=m.source_concat_dim)
            if m.unflatten_dim is not None:
                t = t.unflatten(*m.unflatten_dim)
            if m.dims_permutation is not None:
                t = t.permute(*m.dims_permutation)
            if m.flatten_dims is not None:
                t = t.flatten(*m.flatten_dims)
            for key, piece in zip(m.dest_keys, torch.chunk(t, len(m.dest_keys), dim=m.dest_chunk_dim)):
                out[key] = piece.contiguous()
            leftover.difference_update(m.source_keys)
        if leftover:
            raise RuntimeError(f"Some state keys were not converted: {sorted(leftover)}")
        return out
