"""Experiment configuration trees (``Config``, ``Ref``, ``writable_property``, ``DataClass``)."""
from .core import Config, DataClass, Ref, flatten_dict, recur_to_allowed_types, writable_property
from .arguments import parse_args

__all__ = [
    "Config",
    "DataClass",
    "Ref",
    "writable_property",
    "recur_to_allowed_types",
    "flatten_dict",
    "parse_args",
]
