"""Tree-structured experiment configuration.

The reference builds every experiment out of ``configurize.Config`` trees
(``steptronoss/exp/base_exp.py:39-49``, ``playground/pretrain/qwen3/qwen3_8b.py:102-137``).
``configurize`` is a separate PyPI package; this module is an independent implementation of
the behaviour the reference relies on:

* class-level attributes declare the schema; a value (or annotation default) that is a
  ``Config`` subclass becomes a per-instance child node linked to its parent;
* ``Ref("..a.b", default)`` is a lazy relative link (one leading dot = this node, each further
  dot = one level up);
* ``writable_property`` is a computed attribute that an assignment may override;
* ``merge`` applies dotted-key overrides, ``modify`` is a temporary override context,
  ``sanity_check`` validates recursively, ``to_dict`` serialises the tree.
"""
from __future__ import annotations

import contextlib
import copy
from typing import Any, Iterator

_MISSING = object()


class Ref:
    """Lazy relative reference to another node attribute.

    ``Ref(".x")`` is ``self.x``; ``Ref("..x.y")`` is ``parent.x.y``; ``Ref("...x")`` is
    ``grandparent.x``.  When the path cannot be resolved the ``default`` is returned if one
    was given, otherwise ``AttributeError`` is raised at access time.
    """

    __slots__ = ("path", "default")

    def __init__(self, path: str, default: Any = _MISSING):
        if not path.startswith("."):
            raise ValueError(f"Ref path must start with '.': {path!r}")
        self.path = path
        self.default = default

    def resolve(self, node: "Config") -> Any:
        stripped = self.path.lstrip(".")
        ups = len(self.path) - len(stripped) - 1
        cur: Any = node
        try:
            for _ in range(ups):
                cur = cur.father()
                if cur is None:
                    raise AttributeError(f"Ref {self.path!r}: no ancestor")
            for part in stripped.split("."):
                if part:
                    cur = getattr(cur, part)
        except AttributeError:
            if self.default is not _MISSING:
                return self.default
            raise
        return cur

    def __repr__(self) -> str:
        if self.default is _MISSING:
            return f"Ref({self.path!r})"
        return f"Ref({self.path!r}, {self.default!r})"

    def __deepcopy__(self, memo):
        return Ref(self.path, copy.deepcopy(self.default, memo) if self.default is not _MISSING else _MISSING)


class writable_property:  # noqa: N801  (name is part of the public surface)
    """A property computed from other fields that an assignment may override."""

    def __init__(self, fget):
        self.fget = fget
        self.__doc__ = fget.__doc__
        self.name = fget.__name__

    def __set_name__(self, owner, name):
        self.name = name

    def __get__(self, obj, objtype=None):
        if obj is None:
            return self
        val = obj.__dict__.get("_wp_" + self.name, _MISSING)
        if val is _MISSING:
            return self.fget(obj)
        if isinstance(val, Ref):
            return val.resolve(obj)
        return val

    def __set__(self, obj, value):
        obj.__dict__["_wp_" + self.name] = value

    def __delete__(self, obj):
        obj.__dict__.pop("_wp_" + self.name, None)


def _is_config_class(v: Any) -> bool:
    return isinstance(v, type) and issubclass(v, Config)


class _ConfigMeta(type):
    def __call__(cls, *args, **kwargs):
        obj = cls.__new__(cls)
        d = obj.__dict__
        d["_parent"] = None
        d["_name"] = None
        d["_in_init"] = True
        obj._materialise_declared()
        obj.__init__(*args, **kwargs)
        d["_in_init"] = False
        return obj


class Config(metaclass=_ConfigMeta):
    """Base class of every configuration node."""

    _allow_set_new_attr: bool = False

    def __init__(self) -> None:
        pass

    # ------------------------------------------------------------------ schema
    @classmethod
    def _declared(cls) -> dict[str, Any]:
        """Declared field name -> class-level default (``_MISSING`` when only annotated)."""
        cached = cls.__dict__.get("_declared_cache")
        if cached is not None:
            return cached
        out: dict[str, Any] = {}
        for klass in reversed(cls.__mro__):
            if klass is object:
                continue
            ann = klass.__dict__.get("__annotations__", {})
            for name in ann:
                if name.startswith("_") or name in klass.__dict__:
                    continue
                out.setdefault(name, _MISSING)
            for name, val in klass.__dict__.items():
                if name.startswith("_"):
                    continue
                if hasattr(val, "__get__") and not _is_config_class(val):
                    # functions, properties, cached_property, writable_property, ... are behaviour
                    out.pop(name, None)
                    continue
                out[name] = val
        cls._declared_cache = out
        return out

    def _materialise_declared(self) -> None:
        for name, default in type(self)._declared().items():
            if default is _MISSING:
                continue
            if _is_config_class(default):
                self._attach(name, default())
            elif isinstance(default, Config):
                self._attach(name, copy.deepcopy(default))
            elif isinstance(default, Ref):
                self.__dict__[name] = default
            elif isinstance(default, (dict, list, set)):
                self.__dict__[name] = copy.deepcopy(default)
            # immutable defaults are read through the class attribute

    def _attach(self, name: str, child: "Config") -> None:
        child.__dict__["_parent"] = self
        child.__dict__["_name"] = name
        self.__dict__[name] = child

    # ------------------------------------------------------------ attribute io
    def __getattribute__(self, name: str):
        val = object.__getattribute__(self, name)
        if name[0] != "_" and isinstance(val, Ref):
            return val.resolve(self)
        if name[0] != "_" and _is_config_class(val) and name in type(self)._declared():
            # a class-level child declared after instantiation (rare): materialise lazily
            child = val()
            self._attach(name, child)
            return child
        return val

    def __getattr__(self, name: str):
        if not name.startswith("_") and name in type(self)._declared():
            raise AttributeError(f"{type(self).__name__}.{name} is declared but has no value")
        raise AttributeError(f"{type(self).__name__!s} has no attribute {name!r}")

    def __setattr__(self, name: str, value: Any) -> None:
        if name.startswith("_"):
            self.__dict__[name] = value
            return
        cls_attr = getattr(type(self), name, _MISSING)
        if isinstance(cls_attr, writable_property):
            cls_attr.__set__(self, value)
            return
        if isinstance(cls_attr, property):
            if cls_attr.fset is None:
                raise AttributeError(f"{type(self).__name__}.{name} is a read-only property")
            cls_attr.fset(self, value)
            return
        known = name in type(self)._declared() or name in self.__dict__
        if not known and not (self.__dict__.get("_in_init") or self._allow_set_new_attr):
            raise AttributeError(
                f"{type(self).__name__} has no declared attribute {name!r}; "
                "declare it on the class or set _allow_set_new_attr = True"
            )
        if _is_config_class(value):
            value = value()
        if isinstance(value, Config) and value.__dict__.get("_parent") in (None, self):
            self._attach(name, value)
        else:
            self.__dict__[name] = value

    # ------------------------------------------------------------- navigation
    def father(self) -> "Config | None":
        return self.__dict__.get("_parent")

    def root(self) -> "Config":
        node = self
        while node.father() is not None:
            node = node.father()
        return node

    def _get_node_name(self) -> str:
        parts = []
        node = self
        while node.father() is not None:
            parts.append(node.__dict__.get("_name") or "?")
            node = node.father()
        parts.append(type(node).__name__)
        return ".".join(reversed(parts))

    @property
    def _defined_attributes(self) -> list[str]:
        names = list(type(self)._declared().keys())
        for k in self.__dict__:
            if not k.startswith("_") and k not in names:
                names.append(k)
        return names

    # ------------------------------------------------------- mapping protocol
    def keys(self) -> list[str]:
        return self._defined_attributes

    def items(self) -> Iterator[tuple[str, Any]]:
        for k in self._defined_attributes:
            try:
                yield k, getattr(self, k)
            except AttributeError:
                continue

    def values(self):
        for _, v in self.items():
            yield v

    def __getitem__(self, key: str):
        try:
            return getattr(self, key)
        except AttributeError as e:
            raise KeyError(key) from e

    def __setitem__(self, key: str, value: Any) -> None:
        setattr(self, key, value)

    def __contains__(self, key: str) -> bool:
        return key in self._defined_attributes

    def __iter__(self):
        return iter(self._defined_attributes)

    # --------------------------------------------------------------- utilities
    def _raw(self, name: str) -> Any:
        """Value as stored (a ``Ref`` stays a ``Ref``)."""
        if name in self.__dict__:
            return self.__dict__[name]
        wp = self.__dict__.get("_wp_" + name, _MISSING)
        if wp is not _MISSING:
            return wp
        return type(self)._declared().get(name, _MISSING)

    def _fix_ref(self) -> None:
        """Replace every ``Ref`` below this node by its current value (so the node can be detached)."""
        for k in list(self._defined_attributes):
            raw = self._raw(k)
            if isinstance(raw, Ref):
                try:
                    self.__dict__[k] = raw.resolve(self)
                except AttributeError:
                    pass
            elif isinstance(raw, Config):
                raw._fix_ref()

    @contextlib.contextmanager
    def modify(self, **kwargs):
        """Temporarily assign attributes; the previous raw values come back on exit."""
        saved: dict[str, Any] = {}
        added: list[str] = []
        prev_allow = self.__dict__.get("_allow_set_new_attr", _MISSING)
        self.__dict__["_allow_set_new_attr"] = True
        try:
            for k, v in kwargs.items():
                raw = self._raw(k)
                if raw is _MISSING and k not in self.__dict__:
                    added.append(k)
                else:
                    saved[k] = (k in self.__dict__ or ("_wp_" + k) in self.__dict__, raw)
                setattr(self, k, v)
            yield self
        finally:
            for k in added:
                self.__dict__.pop(k, None)
                self.__dict__.pop("_wp_" + k, None)
            for k, (was_instance, raw) in saved.items():
                self.__dict__.pop(k, None)
                self.__dict__.pop("_wp_" + k, None)
                if was_instance:
                    if isinstance(getattr(type(self), k, None), writable_property):
                        self.__dict__["_wp_" + k] = raw
                    else:
                        self.__dict__[k] = raw
            if prev_allow is _MISSING:
                self.__dict__.pop("_allow_set_new_attr", None)
            else:
                self.__dict__["_allow_set_new_attr"] = prev_allow

    def merge(self, other: "dict | Config", exists_only: bool = False) -> list[tuple[str, Any, Any]]:
        """Apply overrides. Keys may be dotted (``a.b.c``) or nested dicts.

        Returns ``(dotted key, old value, new value)`` for each value that changed.  With
        ``exists_only`` a key that names no existing attribute raises ``KeyError``.
        """
        diff: list[tuple[str, Any, Any]] = []
        if isinstance(other, Config):
            other = other.to_dict()
        for key, value in other.items():
            self._merge_one(key, key, value, exists_only, diff)
        return diff

    def _merge_one(self, full_key, key, value, exists_only, diff):
        head, _, rest = key.partition(".")
        if rest:
            try:
                child = getattr(self, head)
            except AttributeError:
                raise KeyError(f"{full_key}: {type(self).__name__} has no attribute {head!r}") from None
            if isinstance(child, Config):
                child._merge_one(full_key, rest, value, exists_only, diff)
            elif isinstance(child, dict):
                sub = child
                parts = rest.split(".")
                for p in parts[:-1]:
                    sub = sub[p]
                old = sub.get(parts[-1], _MISSING)
                if exists_only and old is _MISSING:
                    raise KeyError(full_key)
                if old != value:
                    diff.append((full_key, None if old is _MISSING else old, value))
                    sub[parts[-1]] = value
            else:
                raise KeyError(f"{full_key}: {head!r} is not a config node")
            return
        exists = head in self._defined_attributes or isinstance(
            getattr(type(self), head, None), (writable_property, property)
        )
        if not exists:
            if exists_only:
                raise KeyError(f"{full_key}: {type(self).__name__} has no attribute {head!r}")
            self.__dict__["_allow_set_new_attr"] = True
        try:
            old = getattr(self, head)
        except AttributeError:
            old = _MISSING
        if isinstance(old, Config) and isinstance(value, dict):
            for k, v in value.items():
                old._merge_one(f"{full_key}.{k}", k, v, exists_only, diff)
            return
        if old is _MISSING or _differs(old, value):
            diff.append((full_key, None if old is _MISSING else old, value))
            setattr(self, head, value)

    def to_dict(self, rep: bool = False) -> dict[str, Any]:
        out: dict[str, Any] = {}
        for k in self._defined_attributes:
            try:
                v = getattr(self, k)
            except Exception:  # unresolved Ref / unset required field
                continue
            if isinstance(v, Config):
                out[k] = v.to_dict(rep=rep)
            elif rep:
                out[k] = repr(v)
            else:
                out[k] = v
        for name in dir(type(self)):
            if isinstance(getattr(type(self), name, None), writable_property) and name not in out:
                try:
                    v = getattr(self, name)
                except Exception:
                    continue
                out[name] = repr(v) if rep else v
        return out

    def sanity_check(self) -> None:
        """Recursive validation: every declared field must have a value; children are checked."""
        for name, default in type(self)._declared().items():
            if default is _MISSING and name not in self.__dict__:
                raise AssertionError(f"{self._get_node_name()}.{name} is required but unset")
        for _, v in list(self.items()):
            if isinstance(v, Config) and v.father() is self:
                v.sanity_check()

    def diff(self, other: "Config") -> list[tuple[str, Any, Any]]:
        """Flattened differences ``(key, mine, theirs)`` between two trees."""
        a, b = flatten_dict(self.to_dict(rep=True)), flatten_dict(other.to_dict(rep=True))
        return [(k, a.get(k), b.get(k)) for k in sorted(set(a) | set(b)) if a.get(k) != b.get(k)]

    _critical_attrs: tuple = ()

    def assert_critical_attrs_expected(self, saved: dict) -> None:
        """Compare a checkpointed ``to_dict`` against this tree on the keys listed in ``_critical_attrs``."""
        mine = flatten_dict(self.to_dict(rep=True))
        theirs = flatten_dict(saved if isinstance(saved, dict) else saved.to_dict(rep=True))
        bad = []
        for k in self._critical_attrs:
            if k in theirs and str(mine.get(k)) != str(theirs[k]):
                bad.append((k, mine.get(k), theirs[k]))
        if bad:
            raise AssertionError("critical config attributes differ from checkpoint: " + repr(bad))

    # ------------------------------------------------------------ presentation
    @staticmethod
    def _brief(v) -> str:
        """``repr`` that never walks into another part of the tree: a config reached through a reference (or a bound
        method of one, e.g. an activation function borrowed from the parent) is named, not printed, which also keeps
        a child that points at its ancestor from recursing for ever."""
        if isinstance(v, Config):
            return f"<{type(v).__name__}>"
        owner = getattr(v, "__self__", None)
        if isinstance(owner, Config):
            return f"<method {type(owner).__name__}.{getattr(v, '__name__', '?')}>"
        return repr(v)

    def format_tree(self, indent: int = 0) -> str:
        pad = "  " * indent
        lines = []
        for k in self._defined_attributes:
            raw = self._raw(k)
            try:
                v = getattr(self, k)
            except Exception as e:
                lines.append(f"{pad}{k}: <unset: {e}>")
                continue
            if isinstance(v, Config) and v.father() is self:
                lines.append(f"{pad}{k}: {type(v).__name__}")
                lines.append(v.format_tree(indent + 1))
            elif isinstance(raw, Ref):
                lines.append(f"{pad}{k}: {self._brief(v)}    <- {raw!r}")
            else:
                lines.append(f"{pad}{k}: {self._brief(v)}")
        return "\n".join(x for x in lines if x)

    def __repr__(self) -> str:
        return f"{type(self).__name__}(\n{self.format_tree(1)}\n)"

    def __deepcopy__(self, memo):
        new = type(self).__new__(type(self))
        memo[id(self)] = new
        for k, v in self.__dict__.items():
            if k == "_parent":
                new.__dict__[k] = memo.get(id(v)) if v is not None else None
            elif isinstance(v, Config) and v.__dict__.get("_parent") is self:
                child = copy.deepcopy(v, memo)
                child.__dict__["_parent"] = new
                new.__dict__[k] = child
            else:
                new.__dict__[k] = copy.deepcopy(v, memo)
        return new

    def __getstate__(self):
        return self.__dict__

    def __setstate__(self, state):
        self.__dict__.update(state)


def _differs(a: Any, b: Any) -> bool:
    try:
        return bool(a != b)
    except Exception:
        return a is not b


def flatten_dict(d: dict, prefix: str = "") -> dict[str, Any]:
    out = {}
    for k, v in d.items():
        key = f"{prefix}{k}"
        if isinstance(v, dict):
            out.update(flatten_dict(v, key + "."))
        else:
            out[key] = v
    return out


class DataClass:
    """Attribute bag with declared fields, mapping access and ``**obj`` unpacking.

    Used for samples that travel through ``broadcast_tensors`` and pickles
    (reference ``steptronoss/exp/rl.py:44-182``).
    """

    def __init__(self, **kwargs):
        for name, default in self._declared_fields().items():
            if default is not _MISSING:
                object.__setattr__(self, name, copy.deepcopy(default))
        for k, v in kwargs.items():
            setattr(self, k, v)

    @classmethod
    def _declared_fields(cls) -> dict[str, Any]:
        out: dict[str, Any] = {}
        for klass in reversed(cls.__mro__):
            if klass in (object, DataClass):
                continue
            for name in klass.__dict__.get("__annotations__", {}):
                if not name.startswith("_"):
                    out[name] = klass.__dict__.get(name, out.get(name, _MISSING))
            for name, val in klass.__dict__.items():
                if name.startswith("_") or callable(val) or isinstance(val, (property, staticmethod, classmethod)):
                    continue
                out[name] = val
        return out

    @property
    def _defined_attributes(self) -> list[str]:
        names = list(self._declared_fields().keys())
        names += [k for k in self.__dict__ if k not in names and not k.startswith("_")]
        return names

    def keys(self):
        return [k for k in self._defined_attributes if hasattr(self, k)]

    def items(self):
        return [(k, getattr(self, k)) for k in self.keys()]

    def values(self):
        return [getattr(self, k) for k in self.keys()]

    def __getitem__(self, key):
        try:
            return getattr(self, key)
        except AttributeError as e:
            raise KeyError(key) from e

    def __setitem__(self, key, value):
        setattr(self, key, value)

    def __contains__(self, key):
        return hasattr(self, key)

    def __iter__(self):
        return iter(self.keys())

    def get(self, key, default=None):
        return getattr(self, key, default)

    def to_dict(self) -> dict[str, Any]:
        return dict(self.items())

    def __eq__(self, other):
        return type(self) is type(other) and self.to_dict() == other.to_dict()

    def __repr__(self):
        body = ", ".join(f"{k}={v!r}" for k, v in self.items())
        return f"{type(self).__name__}({body})"


_PLAIN = (int, float, str, bool, bytes, type(None))


def recur_to_allowed_types(obj: Any) -> Any:
    """Turn a nested object into plain picklable containers (configs and data classes become dicts)."""
    if isinstance(obj, _PLAIN):
        return obj
    if isinstance(obj, Config):
        return {k: recur_to_allowed_types(v) for k, v in obj.to_dict().items()}
    if isinstance(obj, DataClass):
        return {k: recur_to_allowed_types(v) for k, v in obj.items()}
    if isinstance(obj, dict):
        return {recur_to_allowed_types(k): recur_to_allowed_types(v) for k, v in obj.items()}
    if isinstance(obj, (list, tuple, set)):
        return type(obj)(recur_to_allowed_types(v) for v in obj)
    try:
        import torch

        if isinstance(obj, (torch.Tensor, torch.dtype, torch.device)):
            return obj if isinstance(obj, torch.Tensor) else str(obj)
    except ImportError:  # pragma: no cover
        pass
    try:
        import numpy as np

        if isinstance(obj, (np.ndarray, np.generic)):
            return obj
    except ImportError:  # pragma: no cover
        pass
    return repr(obj)
