"""
Import alias: ``import olmo_core.<x>`` resolves to ``olmo_core_b200.<x>`` (the very same module objects), so
scripts written against the reference's package name, ``_CLASS_`` strings in saved configs and pickled
checkpoint metadata work unchanged.
"""

import importlib
import importlib.abc
import importlib.util
import sys

_ALIAS = "olmo_core"
_TARGET = "olmo_core_b200"


class _AliasLoader(importlib.abc.Loader):
    def __init__(self, target_name: str):
        self.target_name = target_name

    def create_module(self, spec):
        return importlib.import_module(self.target_name)

    def exec_module(self, module):
        pass


class _AliasFinder(importlib.abc.MetaPathFinder):
    def find_spec(self, fullname, path=None, target=None):
        if not fullname.startswith(_ALIAS + "."):
            return None
        target_name = _TARGET + fullname[len(_ALIAS):]
        try:
            real = importlib.util.find_spec(target_name)
        except (ImportError, ValueError):
            return None
        if real is None:
            return None
        spec = importlib.util.spec_from_loader(fullname, _AliasLoader(target_name), is_package=real.submodule_search_locations is not None)
        return spec


if not any(isinstance(f, _AliasFinder) for f in sys.meta_path):
    sys.meta_path.insert(0, _AliasFinder())

_real = importlib.import_module(_TARGET)
__path__ = []  # submodules come from the finder above
__version__ = getattr(importlib.import_module(_TARGET + ".version"), "VERSION", "0")
