"""Run every task of a single-node experiment as local process groups."""
from __future__ import annotations

import argparse
import os
import signal
import subprocess
import sys
import time

from .common import expand_tasks, load_exp


def validate(exp) -> list:
    errs = []
    rsc = exp.resource_cfg
    if rsc.replica != 1:
        errs.append("mp_run is single-node: resource_cfg.replica must be 1 (use build_scripts for multi-node runs)")
    for name, spec in rsc.find_leaf_task_specs().items():
        if spec.get("replica", 1) != 1:
            errs.append(f"mp_run is single-node: task '{name}' sets replica={spec.get('replica')}")
    return errs


def _stop(proc: subprocess.Popen, sig=signal.SIGTERM) -> None:
    """Signal the task's own process group (it was started with ``setsid``)."""
    if proc.poll() is None:
        try:
            os.killpg(proc.pid, sig)
        except ProcessLookupError:
            pass


def spawn(tasks: list, poll_s: float = 0.5) -> int:
    procs = [(t, subprocess.Popen(t.command, shell=True, env=os.environ | t.envs, preexec_fn=os.setsid))  # noqa: S602
             for t in tasks]
    critical = [p for t, p in procs if t.is_critical] or [p for _, p in procs]
    rc = 0
    try:
        while any(p.poll() is None for p in critical):
            time.sleep(poll_s)
        rc = max((p.returncode or 0) for p in critical)
    except KeyboardInterrupt:
        rc = 130
    finally:
        for _, p in procs:
            _stop(p)
        deadline = time.time() + 10
        for _, p in procs:
            try:
                p.wait(timeout=max(0.1, deadline - time.time()))
            except subprocess.TimeoutExpired:
                _stop(p, signal.SIGKILL)
    return rc


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description="Run an experiment's tasks on this node.",
                                 epilog="Unrecognised arguments (key=value) are passed to the experiment.")
    ap.add_argument("exp", help="path of the experiment file (defines class Exp)")
    args, extra = ap.parse_known_args(argv)
    exp = load_exp(args.exp, extra)
    errs = validate(exp)
    if errs:
        print("Environment validation failed:\n" + "\n".join(f"  - {e}" for e in errs), file=sys.stderr)
        return 1
    _, tasks = expand_tasks(exp, args.exp, extra)
    for t in tasks:
        print(f"[mp_run] {t.name}: {t.command}")
    return spawn(tasks)


if __name__ == "__main__":
    sys.exit(main())
