"""Abstract configuration nodes that concrete experiments specialise (reference ``steptronoss/exp/abstract.py``)."""
from __future__ import annotations

from ..config import Config


class ModelConfig(Config):
    def build_model(self):
        raise NotImplementedError


class OptimizerConfig(Config):
    def build_optimizer(self, model):
        raise NotImplementedError


class SchedulerConfig(Config):
    lr: float

    def build_scheduler(self, optimizer, *args):
        raise NotImplementedError


class MetricConfig(Config):
    def to_dict(self, rep: bool = False):
        return {k: repr(v) for k, v in self.items()}

    def register_metric(self) -> None:
        """Hook for metric configs that create metrics at run time (the declared ones are registered by ``register``)."""

    def register(self) -> None:
        pass


class TrainerConfig(Config):
    def get_trainer_cls(self):
        raise NotImplementedError


class TokenizerConfig(Config):
    def build_tokenizer(self):
        return None


class DataConfig(Config):
    global_data_keys: list | None = None

    def build_dataloader(self, dp_rank: int = 0, dp_size: int = 1):
        raise NotImplementedError

    def preprocess(self, batch: dict) -> dict:
        return batch
