"""Replace functions by dotted name, for porting experiments that rely on such patches (the reference keeps its
hardware ports as patch lists, ``steptronoss/utils/patch_utils.py:20-127``).

``register_patch("pkg.mod.func", new_func)`` queues a replacement; a callable whose name ends in ``wrapper`` or
``decorator`` is queued as a wrapper around whatever the function is at apply time (several may stack, in
registration order).  ``apply_patches()`` installs everything: on the owning module or class and on every loaded
module that imported the original by name.  ``create_dummy=True`` lets a patch target a module that cannot be
imported here (a stand-in module is created) or a function that does not exist (calling the stand-in raises).
Unlike the reference, ``remove_patches()`` puts the originals back, which tests need.
"""
from __future__ import annotations

import importlib
import sys
import types


def get_func_name(func) -> str:
    return func if isinstance(func, str) else f"{func.__module__}.{func.__qualname__}"


def _missing(name: str):
    def missing(*a, **k):
        raise RuntimeError(f"function {name} does not exist")

    return missing


dummy_function_wrapper = _missing         # the reference's name: a stand-in that raises when called


def _resolve_owner(path: str, create_dummy: bool):
    """Import the longest importable prefix of ``path`` and walk the remaining attributes (classes, sub-objects)."""
    parts = path.split(".")
    owner, used = None, 0
    for i in range(len(parts), 0, -1):
        try:
            owner, used = importlib.import_module(".".join(parts[:i])), i
            break
        except ModuleNotFoundError:
            continue
    if owner is None:
        if not create_dummy:
            raise ModuleNotFoundError(f"cannot import any prefix of {path}")
        used = 0
    for i in range(used, len(parts)):
        name = ".".join(parts[: i + 1])
        nxt = getattr(owner, parts[i], None) if owner is not None else None
        if nxt is None:
            if not create_dummy:
                raise AttributeError(f"{name} does not exist")
            nxt = types.ModuleType(name)
            nxt.__file__ = "<stand-in created by a patch>"
            sys.modules[name] = nxt
            if owner is not None:
                setattr(owner, parts[i], nxt)
        owner = nxt
    return owner


class Patch:
    def __init__(self, target: str, new_func=None, create_dummy: bool = False):
        self.target, self.create_dummy = target, create_dummy
        self.owner_path, _, self.attr = target.rpartition(".")
        self.replacement = None
        self.wrappers: list = []
        self.applied = False
        self._saved: list = []          # (object, attribute, previous value) in the order they were replaced
        self.set_patch_func(new_func if new_func is not None else _missing(target))

    def set_patch_func(self, new_func, force_patch: bool = False) -> None:
        if getattr(new_func, "__name__", "").endswith(("wrapper", "decorator")):
            if new_func not in self.wrappers:
                self.wrappers.append(new_func)
        else:
            if self.replacement is not None and not force_patch:
                raise RuntimeError(f"a patch of {self.target} exists already (pass force_patch=True to replace it)")
            self.replacement = new_func
        self.applied = False

    def apply(self):
        if self.applied:
            return self.installed
        self.remove()
        owner = _resolve_owner(self.owner_path, self.create_dummy) if self.owner_path else None
        if owner is None:
            raise ValueError(f"{self.target} names no attribute of a module")
        sentinel = object()
        original = getattr(owner, self.attr, sentinel)
        if original is sentinel and not self.create_dummy and self.replacement is None:
            raise AttributeError(f"{self.target} does not exist")
        func = self.replacement if self.replacement is not None else original
        for w in self.wrappers:
            func = w(func)
        self._saved.append((owner, self.attr, original))
        setattr(owner, self.attr, func)
        if original is not sentinel and original is not None:
            for mod in list(sys.modules.values()):   # modules that did ``from x import func``
                if mod is owner or not isinstance(mod, types.ModuleType):
                    continue
                try:
                    same = mod.__dict__.get(self.attr) is original
                except Exception:
                    same = False
                if same:
                    self._saved.append((mod, self.attr, original))
                    setattr(mod, self.attr, func)
        self._sentinel = sentinel
        self.installed, self.applied = func, True
        return func

    def remove(self) -> None:
        for obj, attr, prev in reversed(self._saved):
            if prev is getattr(self, "_sentinel", None):
                try:
                    delattr(obj, attr)
                except AttributeError:
                    pass
            else:
                setattr(obj, attr, prev)
        self._saved, self.applied = [], False


class PatchesManager:
    patches_info: dict = {}

    @classmethod
    def register_patch(cls, orig_func_name, new_func=None, force_patch: bool = False, create_dummy: bool = False) -> Patch:
        name = get_func_name(orig_func_name)
        if name not in cls.patches_info:
            cls.patches_info[name] = Patch(name, new_func, create_dummy)
        else:
            cls.patches_info[name].set_patch_func(new_func, force_patch)
        return cls.patches_info[name]

    @classmethod
    def apply_patches(cls) -> None:
        for p in cls.patches_info.values():
            p.apply()

    @classmethod
    def remove_patches(cls, forget: bool = True) -> None:
        for p in reversed(list(cls.patches_info.values())):
            p.remove()
        if forget:
            cls.patches_info = {}


StepTronPatchesManager = PatchesManager   # the reference's name
