"""``import art`` alias of :mod:`art_b200`.

Code written against the reference's package name keeps working: ``import art``,
``from art.local import LocalBackend``, ``from art.utils import iterate_dataset``,
``art.dev.TrainConfig`` ... all resolve to the modules of ``art_b200`` (the same module objects,
not copies).  Reference layout: ``src/art/__init__.py:1-57``.
"""
from __future__ import annotations

import importlib
import importlib.abc
import importlib.util
import sys

import art_b200 as _impl
from art_b200 import *  # noqa: F401,F403

__all__ = getattr(_impl, "__all__", [n for n in dir(_impl) if not n.startswith("_")])
__version__ = getattr(_impl, "__version__", "0")


class _AliasLoader(importlib.abc.Loader):
    def __init__(self, target: str):
        self.target = target

    def create_module(self, spec):
        return importlib.import_module(self.target)

    def exec_module(self, module):   # the real module is already initialised
        pass


class _AliasFinder(importlib.abc.MetaPathFinder):
    def find_spec(self, fullname, path=None, target=None):
        if not fullname.startswith("art."):
            return None
        real = "art_b200." + fullname[4:]
        try:
            if importlib.util.find_spec(real) is None:
                return None
        except ModuleNotFoundError:
            return None
        spec = importlib.util.spec_from_loader(fullname, _AliasLoader(real))
        real_spec = importlib.util.find_spec(real)
        if real_spec is not None and real_spec.submodule_search_locations is not None:
            spec.submodule_search_locations = list(real_spec.submodule_search_locations)
        return spec


if not any(isinstance(f, _AliasFinder) for f in sys.meta_path):
    sys.meta_path.insert(0, _AliasFinder())


def __getattr__(name: str):
    return getattr(_impl, name)
