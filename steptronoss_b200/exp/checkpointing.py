"""Checkpoint configuration (reference ``steptronoss/exp/checkpointing.py:8-108``)."""
from __future__ import annotations

import os

from ..config import Config, Ref, writable_property


class CkptOptions(Config):
    """Which parts of a checkpoint to write / restore: ``opts.none(but=["model"])`` keeps the model only,
    ``opts.all(but=["optimizer"])`` everything but the optimizer."""

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


class SaveOptions(CkptOptions):
    model: bool = True
    optimizer: bool = True
    scheduler: bool = True
    data: bool = True
    rng_state: bool = True


class LoadOptions(CkptOptions):
    model: bool = True
    optimizer: bool = True
    scheduler: bool = True
    data: bool = True
    rng_state: bool = True
    exp: bool = False
    iter: bool = True


class CheckpointConfig(Config):
    save_dir: str = "./checkpoints"
    exp_name = Ref("..exp_name", "exp")
    save_interval: int | None = None
    save_option: SaveOptions = SaveOptions
    save_safetensors: bool = False
    """also write the HF view of the weights to ``<iteration dir>/hf``"""
    async_dump: bool = True
    load_path: str | None = None
    load_safetensors: bool | str | None = None
    """a HF checkpoint directory to take the weights from (``True``: ``<load_path>/hf``)"""
    auto_resume: bool = True
    load_option: LoadOptions = LoadOptions
    broadcast_from_dp0: bool = True
    strict_load_model: bool = True
    use_distributed_optimizer = Ref("..optimizer_cfg.use_distributed_optimizer", False)
    reshard_optimizer_state: bool = False
    reshard_optimizer_strict: bool = True
    model_config_path: str | None = None
    """directory whose ``*.json`` / tokenizer files are copied next to exported safetensors"""
    tokenizer_path: str | None = None
    keep_last: int | None = None

    # earlier spellings of this repository
    @property
    def load_options(self) -> LoadOptions:
        return self.load_option

    @load_options.setter
    def load_options(self, value) -> None:
        self.load_option = value

    @property
    def async_save(self) -> bool:
        return self.async_dump

    @async_save.setter
    def async_save(self, value: bool) -> None:
        self.async_dump = value

    @writable_property
    def save_path(self) -> str:
        return os.path.join(self.save_dir, self.exp_name)

    def sanity_check(self) -> None:
        super().sanity_check()
        if self.load_safetensors and self.load_path and self.load_safetensors is not True:
            raise AssertionError("load_safetensors and load_path cannot be set at the same time")

    def build_checkpointer(self):
        from ..checkpointing.local_checkpoint import Checkpointer

        return Checkpointer(self)
