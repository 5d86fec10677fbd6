"""Trainer skeleton with hook points (reference ``steptronoss/core/trainers/base_trainer.py``)."""
from __future__ import annotations

from typing import Callable


class BaseTrainer:
    def __init__(self, exp):
        self.exp = exp
        self.iteration = 0
        self._hooks: dict[str, list[Callable]] = {"after_init": [], "before_train": [], "before_step": [],
                                                  "after_step": [], "after_train": []}
        self._hooks_built = False

    def register_hook(self, where: str, fn: Callable) -> None:
        self._hooks[where].append(fn)

    def build_hooks(self, trainer_cfg) -> None:
        """Take the hooks that the trainer config builds (``build_after_init_hooks`` ... ``build_after_train_hooks``,
        each a list of ``fn(trainer)``); an experiment overrides those methods to run its own code at the five
        points.  Reference: core/trainers/base_trainer.py:17-22.  Runs once per trainer."""
        if self._hooks_built:
            return
        self._hooks_built = True
        for where in self._hooks:
            build = getattr(trainer_cfg, f"build_{where}_hooks", None)
            if build is not None:
                self._hooks[where].extend(build() or [])

    def call_hooks(self, where: str) -> None:
        for fn in self._hooks[where]:
            fn(self)

    def before_train(self):
        raise NotImplementedError

    def train_loop(self):
        raise NotImplementedError

    def after_train(self):
        pass

    def train(self):
        self.before_train()
        try:
            self.train_loop()
        finally:
            self.after_train()
