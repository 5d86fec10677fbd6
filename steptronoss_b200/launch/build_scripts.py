"""Write one shell script per task replica of an experiment: ``<out>/<exp name>/<exp id>/<node type>/<i>.sh``."""
from __future__ import annotations

import argparse
import os
import shlex
import stat
import sys
from dataclasses import dataclass

from .common import expand_tasks, load_exp


@dataclass(frozen=True)
class BuildScriptsResult:
    exp_id: str
    output_dir: str
    scripts: list


def script_text(envs: dict, command: str) -> str:
    keys = (["EXP_ID"] if "EXP_ID" in envs else []) + sorted(k for k in envs if k != "EXP_ID")
    lines = ["#!/usr/bin/env bash", "set -e", *[f"export {k}={shlex.quote(str(envs[k]))}" for k in keys], command, ""]
    return "\n".join(lines)


def build_scripts(exp_path: str, output_root: str, extra_args: list, exp_id: str | None = None,
                  interactive: bool = True) -> BuildScriptsResult:
    exp = load_exp(exp_path, extra_args, interactive)
    exp_id, tasks = expand_tasks(exp, exp_path, extra_args, exp_id)
    out_dir = os.path.join(output_root, exp.exp_name, exp_id)
    scripts, next_idx = [], {}
    for t in tasks:
        node_dir = os.path.join(out_dir, t.node_type)
        os.makedirs(node_dir, exist_ok=True)
        for _ in range(t.replica):
            i = next_idx.get(t.node_type, 0)
            next_idx[t.node_type] = i + 1
            path = os.path.join(node_dir, f"{i}.sh")
            with open(path, "w", encoding="utf-8") as f:
                f.write(script_text(t.envs, t.command))
            os.chmod(path, os.stat(path).st_mode | stat.S_IXUSR)
            scripts.append(path)
    return BuildScriptsResult(exp_id, out_dir, scripts)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description="Generate per-replica shell scripts for an experiment.")
    ap.add_argument("exp")
    ap.add_argument("output_root")
    args, extra = ap.parse_known_args(argv)
    res = build_scripts(args.exp, args.output_root, extra)
    print(f"Scripts written to: {res.output_dir}")
    print("\n".join(res.scripts))
    return 0


if __name__ == "__main__":
    sys.exit(main())
