"""
Declarative description of how named state in one format maps to named state in another
(API of src/olmo_core/nn/conversion/state_mapping.py:7-280).

A :class:`StateMappingTemplate` names source and destination keys that may contain the placeholders ``[layer]`` and
``[expert]``. Given concrete values it becomes a :class:`StateMapping`: N source tensors are concatenated along
``source_concat_dim``, optionally unflattened / permuted / flattened, then split evenly along ``dest_chunk_dim`` into
the destination keys. A template can also fan a placeholder out over ALL its values on one side
(``source_key_per_placeholder`` / ``dest_key_per_placeholder``), e.g. one stacked expert matrix ↔ one matrix per expert.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional, Tuple, Union

from ...config import StrEnum

__all__ = ["TemplatePlaceholder", "StateType", "StateMappingTemplate", "StateMapping"]


class TemplatePlaceholder(StrEnum):
    LAYER = "[layer]"
    EXPERT = "[expert]"


class StateType(StrEnum):
    weight = "weight"  # the mapped things are parameters (checkpoint conversion)
    module = "module"  # the mapped things are sub-modules (comparing activations of two implementations)


Keys = Union[str, Tuple[str, ...]]


@dataclass
class StateMapping:
    source_keys: Tuple[str, ...]
    dest_keys: Tuple[str, ...]
    state_type: StateType = StateType.weight
    source_concat_dim: int = 0
    unflatten_dim: Optional[Tuple[int, Tuple[int, ...]]] = None
    dims_permutation: Optional[Tuple[int, ...]] = None
    flatten_dims: Optional[Tuple[int, int]] = None
    dest_chunk_dim: int = 0


@dataclass
class StateMappingTemplate:
    source_template_keys: Keys
    dest_template_keys: Keys
    state_type: StateType = StateType.weight
    source_key_per_placeholder: Optional[TemplatePlaceholder] = None
    dest_key_per_placeholder: Optional[TemplatePlaceholder] = None
    source_concat_dim: int = 0
    unflatten_dim: Optional[Tuple[int, Tuple[Union[TemplatePlaceholder, int], ...]]] = None
    dims_permutation: Optional[Tuple[int, ...]] = None
    flatten_dims: Optional[Tuple[int, int]] = None
    dest_chunk_dim: int = 0

    def __post_init__(self):
        for side, fan, keys in (("source", self.source_key_per_placeholder, self.source_template_keys),
                                ("dest", self.dest_key_per_placeholder, self.dest_template_keys)):
            if fan is not None and not isinstance(keys, str):
                raise ValueError(f"fanning {fan} out over the {side} keys needs exactly one {side} template key")

    def _expand(self, templates: Keys, fan: Optional[TemplatePlaceholder], values: Dict[TemplatePlaceholder, Optional[int]],
                bounds: Dict[TemplatePlaceholder, int]) -> Optional[Tuple[str, ...]]:
        if fan is not None:
            assert isinstance(templates, str)
            if str(fan) not in templates:
                raise ValueError(f"placeholder {fan} is fanned out but absent from template '{templates}'")
            if fan not in bounds:
                raise ValueError(f"placeholder {fan} has no bound")
            templates = tuple(templates.replace(str(fan), str(i)) for i in range(bounds[fan]))
        elif isinstance(templates, str):
            templates = (templates,)
        keys = []
        for template in templates:
            for placeholder, value in values.items():
                present = str(placeholder) in template
                if present != (value is not None):
                    return None  # a value for a placeholder the key lacks (or the reverse): not this combination
                if present:
                    template = template.replace(str(placeholder), str(value))
            if any(str(p) in template for p in TemplatePlaceholder):
                return None
            keys.append(template)
        return tuple(keys)

    def to_mapping(self, placeholder_values: Dict[TemplatePlaceholder, Optional[int]],
                   placeholder_bounds: Dict[TemplatePlaceholder, int]) -> Optional[StateMapping]:
        """Concrete mapping for one combination of placeholder values, or ``None`` if the combination does not apply."""
        needed = {p for p in (self.source_key_per_placeholder, self.dest_key_per_placeholder) if p is not None}
        if self.unflatten_dim is not None:
            needed |= {d for d in self.unflatten_dim[1] if isinstance(d, TemplatePlaceholder)}
        if needed - set(placeholder_bounds):
            return None  # e.g. an expert mapping applied to a dense model
        src = self._expand(self.source_template_keys, self.source_key_per_placeholder, placeholder_values, placeholder_bounds)
        dst = self._expand(self.dest_template_keys, self.dest_key_per_placeholder, placeholder_values, placeholder_bounds)
        if src is None or dst is None:
            return None
        unflatten = None
        if self.unflatten_dim is not None:
            shape = tuple(placeholder_bounds[d] if isinstance(d, TemplatePlaceholder) else int(d) for d in self.unflatten_dim[1])
            unflatten = (self.unflatten_dim[0], shape)
        return StateMapping(src, dst, state_type=self.state_type, source_concat_dim=self.source_concat_dim,
                            unflatten_dim=unflatten, dims_permutation=self.dims_permutation,
                            flatten_dims=self.flatten_dims, dest_chunk_dim=self.dest_chunk_dim)
