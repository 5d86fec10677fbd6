"""Stand-in for the ``configurize`` PyPI package (not installable offline) so that the unmodified
reference can be imported for the baseline arm of ``bench.py``.  It exposes this repository's own
implementation of the same configuration-tree API."""
from steptronoss_b200.config import Config, DataClass, Ref, recur_to_allowed_types, writable_property  # noqa: F401

__version__ = "0.2.0"
