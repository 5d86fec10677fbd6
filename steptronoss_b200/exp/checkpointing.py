"""Checkpoint configuration (reference ``steptronoss/exp/checkpointing.py:8-108``)."""
from __future__ import annotations

import os

from ..config import Config, Ref, writable_property


class LoadOptions(Config):
    """Which parts of a checkpoint to restore."""

    model: bool = True
    optimizer: bool = True
    scheduler: bool = True
    data: bool = True
    rng_state: bool = True
    exp: bool = False
    iter: bool = True

    def _names(self):
        return [k for k, v in self.items() if isinstance(v, bool)]

    def all(self, but=()):
        for k in self._names():
            setattr(self, k, k not in but)
        return self

    def none(self, but=()):
        for k in self._names():
            setattr(self, k, k in but)
        return self


class CheckpointConfig(Config):
    save_dir: str = "./checkpoints"
    exp_name = Ref("..exp_name", "exp")
    save_interval: int | None = None
    save_safetensors: bool = False
    async_save: bool = True
    load_path: str | None = None
    load_safetensors: str | None = None
    auto_resume: bool = True
    load_options: LoadOptions = LoadOptions
    reshard_optimizer_state: bool = False
    keep_last: int | None = None

    @writable_property
    def save_path(self) -> str:
        return os.path.join(self.save_dir, self.exp_name)

    def build_checkpointer(self):
        from ..checkpointing.local_checkpoint import Checkpointer

        return Checkpointer(self)
