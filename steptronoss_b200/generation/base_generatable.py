"""Units of generation work (reference ``steptronoss/generation/base_generatable.py:9-65``).

A :class:`GenableItem` knows how to produce its own output (usually by calling the experiment's inference
router); a :class:`TrainableItem` additionally turns that output into rewarded trajectories.  Items are
pickled to worker processes, so they carry *getters* for the router endpoint and the served model name
instead of concrete strings: both can change between a run and its resume.
"""
from __future__ import annotations

from abc import ABC, abstractmethod
from typing import Any


class GenableItem(ABC):
    def __init__(self, meta: dict | None = None) -> None:
        self.meta: dict = meta or {}

    @abstractmethod
    async def generate(self) -> Any:
        ...

    def fingerprint(self) -> str:
        """Stable cache key of this request; items that take part in persistent caching override it."""
        raise NotImplementedError(f"{type(self).__name__} must implement fingerprint() for generation caching")


class TrainableItem(GenableItem):
    @abstractmethod
    async def generate_for_train(self) -> list:
        """Return a list of :class:`steptronoss_b200.exp.rl.EnvTrajectory`."""


class EndpointGetter:
    """Resolve the router's ``http://host:port`` at call time from the experiment store."""

    def __init__(self, router_addr_key: str):
        self.router_addr_key = router_addr_key

    def __call__(self) -> str:
        from ..utils.comm_utils import block_get_redis, get_exp_redis

        key = f"VLLM_ROUTER_ADDR_PORT_{self.router_addr_key}"
        return f"http://{block_get_redis(get_exp_redis(), key).decode()}"


class ModelNameGetter:
    """Resolve the served model name (it embeds the experiment id) at call time."""

    def __init__(self, model_name_template: str):
        self.model_name_template = model_name_template

    def __call__(self) -> str:
        from ..utils.comm_utils import get_exp_id

        return self.model_name_template.format(EXP_ID=get_exp_id())
