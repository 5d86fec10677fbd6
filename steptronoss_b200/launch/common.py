"""Shared pieces of the launchers: load the ``Exp`` class of a file, apply CLI overrides, expand tasks."""
from __future__ import annotations

import importlib.util
import os
import shlex
import sys
import traceback
from dataclasses import dataclass, field
from uuid import uuid4

SMARTRUN = f"{shlex.quote(sys.executable)} -m steptronoss_b200.launch.smartrun"


def get_object_from_file(path: str, name: str = "Exp"):
    """Import ``path`` as a module (the working directory is importable, as for ``python path``) and return
    its attribute ``name``."""
    path = os.path.abspath(path)
    if os.getcwd() not in sys.path:
        sys.path.insert(0, os.getcwd())
    mod_name = "_exp_" + os.path.splitext(os.path.basename(path))[0]
    spec = importlib.util.spec_from_file_location(mod_name, path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules[mod_name] = mod
    spec.loader.exec_module(mod)
    return getattr(mod, name)


@dataclass
class Task:
    name: str
    command: str
    envs: dict
    replica: int
    node_type: str
    is_critical: bool
    extra: dict = field(default_factory=dict)


def load_exp(exp_path: str, extra_args: list, interactive: bool = True):
    """Instantiate, apply ``key=value`` overrides, sanity-check (a failure can be waved through)."""
    exp = get_object_from_file(exp_path, "Exp")()
    exp.update_from_args(list(extra_args))
    try:
        exp.sanity_check()
    except Exception as e:
        msg = "".join(traceback.format_exception(e)[-2:])
        if interactive and sys.stdin is not None and sys.stdin.isatty():
            input(f"Sanity check failed:\n{msg}\npress enter to ignore and continue")
        else:
            print(f"Sanity check failed (continuing):\n{msg}", file=sys.stderr)
    return exp


def expand_tasks(exp, exp_path: str, extra_args: list, exp_id: str | None = None) -> tuple[str, list]:
    """``(exp_id, tasks)``: one :class:`Task` per entry of the experiment's ``task_specs``."""
    exp_id = exp_id or os.environ.get("EXP_ID") or str(uuid4())[:5]
    os.environ["EXP_ID"] = exp_id
    rsc = exp.resource_cfg
    rsc.envs["EXP_ID"] = exp_id
    command = " ".join([exp_path, *extra_args])
    tasks = []
    for name, cfg in rsc.extract().items():
        tasks.append(Task(name, cfg.command.format(TORCHRUN=SMARTRUN, COMMAND=command),
                          {k: str(v) for k, v in (cfg.envs | {"NNODES": str(cfg.replica)}).items()},
                          int(cfg.replica), cfg.node_type, bool(cfg.is_critical),
                          extra={"image": cfg.image, "mounts": list(cfg.mounts), "gpu": int(cfg.gpu)}))
    return exp_id, tasks
