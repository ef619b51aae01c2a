from typing import Callable, TypeVar

T = TypeVar("T", bound=Callable)


def beta_feature(f: T) -> T:
    """Mark a function or class as a beta feature in its docstring."""
    doc = f.__doc__ or ""
    f.__doc__ = doc + "\n\n.. warning::\n    This is a beta feature; its API may change.\n"
    return f
