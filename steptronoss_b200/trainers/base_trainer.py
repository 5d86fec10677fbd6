"""Trainer skeleton with hook points (reference ``steptronoss/core/trainers/base_trainer.py``)."""
from __future__ import annotations

from typing import Callable


class BaseTrainer:
    def __init__(self, exp):
        self.exp = exp
        self.iteration = 0
        self._hooks: dict[str, list[Callable]] = {"after_init": [], "before_step": [], "after_step": [], "after_train": []}

    def register_hook(self, where: str, fn: Callable) -> None:
        self._hooks[where].append(fn)

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
