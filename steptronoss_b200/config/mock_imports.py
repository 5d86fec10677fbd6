"""Import an experiment file on a machine that lacks the heavy runtime dependencies.

Counterpart of ``configurize.mock_imports`` / ``configurize.utils.get_object_from_file`` as used
by the reference submitter (``tools/example_submitter.py:10-11,75-76``).
"""
from __future__ import annotations

import contextlib
import importlib.abc
import importlib.machinery
import importlib.util
import sys
import types
from pathlib import Path


class _Anything(types.ModuleType):
    """Module stand-in: every attribute is another stand-in, calls return a stand-in."""

    def __getattr__(self, name):
        if name.startswith("__") and name.endswith("__"):
            raise AttributeError(name)
        child = _Anything(f"{self.__name__}.{name}")
        setattr(self, name, child)
        return child

    def __call__(self, *a, **k):
        return _Anything(self.__name__ + "()")

    def __mro_entries__(self, bases):
        return (object,)

    def __iter__(self):
        return iter(())


class _MockFinder(importlib.abc.MetaPathFinder, importlib.abc.Loader):
    def __init__(self, prefixes):
        self.prefixes = tuple(prefixes)

    def find_spec(self, fullname, path, target=None):
        if fullname.split(".")[0] in self.prefixes:
            return importlib.machinery.ModuleSpec(fullname, self, is_package=True)
        return None

    def create_module(self, spec):
        m = _Anything(spec.name)
        m.__path__ = []
        return m

    def exec_module(self, module):
        pass


@contextlib.contextmanager
def mock_imports(*prefixes: str):
    """Within the context, ``import <prefix>...`` yields inert stand-in modules when the real
    package cannot be imported."""
    missing = []
    for p in prefixes:
        if importlib.util.find_spec(p) is None:
            missing.append(p)
    finder = _MockFinder(missing)
    sys.meta_path.append(finder)
    try:
        yield
    finally:
        sys.meta_path.remove(finder)
        for name in [n for n in sys.modules if n.split(".")[0] in missing]:
            del sys.modules[name]


def get_object_from_file(path: str, name: str = "Exp"):
    """Execute the Python file at ``path`` as a module and return its attribute ``name``."""
    path = str(Path(path).resolve())
    mod_name = "_exp_file_" + Path(path).stem
    spec = importlib.util.spec_from_file_location(mod_name, path)
    module = importlib.util.module_from_spec(spec)
    sys.modules[mod_name] = module
    spec.loader.exec_module(module)
    return getattr(module, name)
