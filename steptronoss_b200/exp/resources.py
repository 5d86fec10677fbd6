"""Resource description of the tasks an experiment launches (reference ``steptronoss/exp/resources.py``)."""
from __future__ import annotations

import copy
import os
from typing import TypedDict

from ..config import Config


class TaskSpec(TypedDict, total=False):
    replica: int
    gpu: int
    command: str
    node_type: str
    is_critical: bool
    mounts: list
    envs: dict
    image: str


class ResourceConfig(Config):
    replica: int
    gpu: int
    node_type: str
    is_critical: bool = False
    mounts: list = []
    envs: dict = {}
    image: str | None = None
    command: str

    def __init__(self):
        super().__init__()
        self.task_specs = dict(default=TaskSpec(is_critical=True))
        self.replica = 1
        self.gpu = 0
        self.node_type = "cpu"
        self.command = "python {COMMAND}"

    def extract(self) -> dict:
        """Flatten ``task_specs`` (found anywhere in the tree) into one ResourceConfig per task.

        Each result gets ``exp_name`` and ``envs["EXP_ID"] = "<exp id>/<task>"``."""
        assert isinstance(self.task_specs, dict), self.task_specs
        if "PYTHONPATH" not in self.envs:
            self.envs["PYTHONPATH"] = "."
        specs = self.find_leaf_task_specs()
        exp_id = os.environ["EXP_ID"]
        out = {}
        for task_name, spec in specs.items():
            spec = dict(spec)
            spec["envs"] = self.envs | spec.get("envs", {})
            with self.modify(**spec):
                cfg = self.__class__()
                for k, v in self.items():
                    if k != "task_specs":
                        setattr(cfg, k, copy.deepcopy(v))
                cfg._fix_ref()
                cfg._allow_set_new_attr = True
                cfg.envs["EXP_ID"] = f"{exp_id}/{task_name}"
                root = self.root()
                cfg.exp_name = f"{getattr(root, 'exp_name', 'exp')}/{task_name}"
                out[task_name] = cfg
        return out

    def find_leaf_task_specs(self) -> dict:
        node = self
        while node.father() is not None:
            node = node.father()
            if hasattr(node, "resource_cfg") and isinstance(node.resource_cfg, ResourceConfig):
                break
        found, where = {}, {}

        def walk(n: Config):
            specs = n.__dict__.get("task_specs")
            if isinstance(specs, dict):
                prefix = n._get_node_name()
                for k, v in specs.items():
                    if k in found and v != found[k]:
                        raise RuntimeError(f"Conflict sub-task name '{k}' in {prefix} and {where[k]}!")
                    found[k], where[k] = v, prefix
            for _k, v in n.items():
                if isinstance(v, Config) and v.father() is n:
                    walk(v)

        walk(node)
        return found


class TorchrunResourceConfig(ResourceConfig):
    def __init__(self):
        super().__init__()
        self.node_type = "gpu"
        self.gpu = 8
        self.command = "{TORCHRUN} {COMMAND}"
