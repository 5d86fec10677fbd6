"""``cfshow exp.py [-k subtree] [--diff [other.py]]``: print an experiment's config tree and run its
``sanity_check`` (reference ``README.md:38-45``).  ``--diff`` without a file compares with the experiment class
this one derives from (what the file changes on top of its base)."""
from __future__ import annotations

import argparse
import sys

from .core import Config
from .mock_imports import get_object_from_file


def show(path: str, key: str | None = None, diff: str | None = None, check: bool = True, out=None) -> int:
    out = out or sys.stdout
    exp = get_object_from_file(path, "Exp")()
    node = exp
    if key:
        for part in key.split("."):
            node = getattr(node, part)
    if isinstance(node, Config):
        print(f"{type(node).__name__} @ {node._get_node_name()}", file=out)
        print(node.format_tree(1), file=out)
    else:
        print(repr(node), file=out)
    if diff:
        if diff == "parent":
            bases = [b for b in type(exp).__mro__[1:] if isinstance(b, type) and issubclass(b, Config) and b is not Config]
            if not bases:
                print("--- no parent experiment to diff against", file=out)
                other = None
            else:
                other, diff = bases[0](), f"{bases[0].__module__}.{bases[0].__qualname__}"
        else:
            other = get_object_from_file(diff, "Exp")()
        if other is not None:
            print(f"--- diff vs {diff} (this | other)", file=out)
            for k, a, b in exp.diff(other):
                print(f"  {k}: {a} | {b}", file=out)
    if check:
        try:
            exp.sanity_check()
            print("sanity_check: OK", file=out)
        except Exception as e:  # report, do not hide
            print(f"sanity_check: FAILED: {type(e).__name__}: {e}", file=out)
            return 1
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="cfshow", description=__doc__)
    ap.add_argument("exp_file")
    ap.add_argument("-k", "--key", default=None, help="dotted path of the subtree to print")
    ap.add_argument("--diff", nargs="?", const="parent", default=None,
                    help="another experiment file to diff against; without a value: the parent experiment class")
    ap.add_argument("--no-check", action="store_true")
    ns, rest = ap.parse_known_args(argv)
    sys.argv = [ns.exp_file] + rest
    return show(ns.exp_file, ns.key, ns.diff, check=not ns.no_check)


if __name__ == "__main__":
    raise SystemExit(main())
