"""Template for submitting an experiment to a cluster scheduler.

An experiment's ``resource_cfg`` describes one or more tasks (trainer, rollout servers, ...); each has a node
type, a replica count, an image, mounts, environment variables and a command.  This module turns that description
into calls of ONE function, :meth:`Submitter.launch_task`, which is the only part that depends on the scheduler
(Kubernetes, Slurm, an in-house platform).  Subclass :class:`Submitter`, implement ``launch_task`` (and, when the
scheduler can tell, ``is_running`` / ``terminate``), and call ``run()``.

Same role as the reference's ``tools/example_submitter.py:14-112`` (``launch_task`` left to the user,
``spawn_tasks`` over ``resource_cfg.extract()``, wait on the critical tasks, then stop the rest).

The experiment file is imported with the heavy packages stubbed out where they are missing, so the submitting
machine needs neither a GPU nor torch.
"""
from __future__ import annotations

import argparse
import os
import sys
import time
from dataclasses import dataclass, field

from ..config.mock_imports import mock_imports
from .common import Task, expand_tasks, load_exp

# packages an experiment file may import that a submit host often lacks
HEAVY_PACKAGES = ("torch", "transformers", "vllm", "flash_attn", "safetensors", "tensorboardX", "wandb")


@dataclass
class Submission:
    """What ``launch_task`` gets: one task of the experiment, fully resolved."""
    task: Task
    image: str | None
    mounts: list
    gpus_per_node: int
    code_dir: str
    handle: object = None              # whatever launch_task returned (a job id, a Popen, ...)
    extra: dict = field(default_factory=dict)


class Submitter:
    """Scheduler-independent part of a submission.  ``launch_task`` is the adaptation point."""

    #: where rank 0 of a task publishes its address for the other nodes (a shared directory); exported to the
    #: tasks as ``STEPTRON_MEET_DIR`` and read by the rendezvous in ``utils.comm_utils``
    meet_dir: str | None = None
    poll_s: float = 5.0

    def __init__(self, exp_path: str, exp_args: list | None = None, image: str | None = None,
                 code_dir: str | None = None, interactive: bool = True):
        self.exp_path = exp_path
        self.exp_args = list(exp_args or [])
        self.image = image
        self.code_dir = code_dir or os.getcwd()
        self.interactive = interactive

    # ------------------------------------------------------------------ to implement
    def launch_task(self, sub: Submission):
        """Start ``sub.task.replica`` nodes of type ``sub.task.node_type`` that run ``sub.task.command`` with
        ``sub.task.envs`` in image ``sub.image`` with ``sub.code_dir`` as the working directory.  Return a handle."""
        raise NotImplementedError(
            "adapt Submitter.launch_task to your scheduler: it receives the command, environment, image, mounts, "
            "node type and replica count of one task")

    def is_running(self, sub: Submission) -> bool:
        """Whether the task is still alive.  The default understands ``subprocess.Popen`` handles."""
        h = sub.handle
        if hasattr(h, "poll"):
            return h.poll() is None
        return False

    def terminate(self, sub: Submission) -> None:
        h = sub.handle
        if hasattr(h, "terminate") and self.is_running(sub):
            h.terminate()

    # ------------------------------------------------------------------ fixed part
    def load(self):
        with mock_imports(*HEAVY_PACKAGES):
            return load_exp(self.exp_path, self.exp_args, interactive=self.interactive)

    def resolve(self, exp, exp_id: str | None = None) -> list:
        """One :class:`Submission` per task of the experiment."""
        exp_id, tasks = expand_tasks(exp, self.exp_path, self.exp_args, exp_id)
        out = []
        for task in tasks:
            if self.meet_dir:
                task.envs["STEPTRON_MEET_DIR"] = os.path.join(self.meet_dir, exp_id, task.name)
            out.append(Submission(task, task.extra["image"] or self.image, task.extra["mounts"], task.extra["gpu"],
                                  self.code_dir))
        return out

    def spawn_tasks(self, subs: list) -> list:
        for s in subs:
            print(f"[submit] {s.task.name}: {s.task.replica} x {s.task.node_type} ({s.gpus_per_node} GPUs/node)"
                  f"{' [critical]' if s.task.is_critical else ''}\n         {s.task.command}")
            s.handle = self.launch_task(s)
        return subs

    def wait(self, subs: list) -> None:
        """Return when no critical task is running any more (all tasks count when none is marked), then stop the
        others: rollout servers and the like have no end of their own."""
        critical = [s for s in subs if s.task.is_critical] or subs
        try:
            while any(self.is_running(s) for s in critical):
                time.sleep(self.poll_s)
        finally:
            for s in subs:
                self.terminate(s)

    def run(self, wait: bool = True) -> list:
        exp = self.load()
        subs = self.spawn_tasks(self.resolve(exp))
        if wait:
            self.wait(subs)
        return subs


def main(argv=None, submitter_cls=Submitter) -> int:
    ap = argparse.ArgumentParser(description=__doc__.splitlines()[0],
                                 epilog="Unrecognised arguments (key=value) are passed to the experiment.")
    ap.add_argument("exp", help="path of the experiment file (defines class Exp)")
    ap.add_argument("--image", default=None, help="container image for tasks that name none")
    ap.add_argument("--code-dir", default=None, help="directory the tasks start in (default: the current one)")
    ap.add_argument("--meet-dir", default=None, help="shared directory for the multi-node rendezvous")
    ap.add_argument("--no-wait", action="store_true", help="return right after submission")
    args, extra = ap.parse_known_args(argv)
    sub = submitter_cls(args.exp, extra, image=args.image, code_dir=args.code_dir)
    sub.meet_dir = args.meet_dir
    sub.run(wait=not args.no_wait)
    return 0


if __name__ == "__main__":
    sys.exit(main())
