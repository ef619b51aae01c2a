"""Small enums shared by the data layer (src/olmo_core/data/types.py)."""

from typing import Type, Union

import numpy as np

from ..config import StrEnum

__all__ = ["NumpyUIntTypes", "LongDocStrategy", "NumpyDatasetDType"]

NumpyUIntTypes = Union[Type[np.uint8], Type[np.uint16], Type[np.uint32], Type[np.uint64]]


class LongDocStrategy(StrEnum):
    """What packing does with a document longer than the sequence length."""

    truncate = "truncate"
    """Keep the first ``sequence_length`` tokens, drop the rest."""
    fragment = "fragment"
    """Split into ``sequence_length``-sized pieces; nothing is dropped but pieces lose their left context."""


class NumpyDatasetDType(StrEnum):
    """Token-id storage types of ``.npy`` token files."""

    uint8, uint16, uint32, uint64 = "uint8", "uint16", "uint32", "uint64"

    def as_np_dtype(self) -> NumpyUIntTypes:
        """The numpy scalar type of the same name."""
        return {"uint8": np.uint8, "uint16": np.uint16, "uint32": np.uint32, "uint64": np.uint64}[self.value]
