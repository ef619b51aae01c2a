from os import PathLike
from typing import Union

__all__ = ["PathOrStr"]

PathOrStr = Union[str, "PathLike[str]"]
