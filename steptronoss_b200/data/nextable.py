"""Resumable iterators (reference ``steptronoss/data/nextable/nextable.py:11-102``).

``Nextable``: ``next()`` + ``state_dict`` / ``load_state_dict``.  ``SlowFastNextable`` adds ``fast_step``:
advance the state without producing the item, which is how data-parallel ranks skip each other's samples.
``LazyUpdateNextable`` splits ``next`` into ``get`` (produce from the current state) and ``update`` (advance).
``DPMux`` turns one global stream into the stream of DP rank ``r``: item ``i`` belongs to rank ``i % dp_size``.
"""
from __future__ import annotations

from abc import ABCMeta, abstractmethod
from typing import Any


class Nextable(metaclass=ABCMeta):
    def __iter__(self):
        return self

    @abstractmethod
    def __next__(self) -> Any: ...

    @abstractmethod
    def state_dict(self) -> dict: ...

    @abstractmethod
    def load_state_dict(self, state: dict) -> None: ...

    @classmethod
    def __subclasshook__(cls, sub):
        if cls is Nextable:
            return all(callable(getattr(sub, n, None)) for n in ("__next__", "state_dict", "load_state_dict"))
        return NotImplemented


class SlowFastNextable(Nextable):
    @abstractmethod
    def fast_step(self) -> None:
        """Advance exactly as ``next`` would, without building the item."""


class LazyUpdateNextable(SlowFastNextable):
    @abstractmethod
    def get(self) -> Any: ...

    @abstractmethod
    def update(self) -> None: ...

    def fast_step(self) -> None:
        self.update()

    def __next__(self):
        item = self.get()
        self.update()
        return item


class DPMux(SlowFastNextable):
    def __init__(self, slowfast: SlowFastNextable, dp_size: int = 1, dp_rank: int = 0):
        self.inner, self.dp_size, self.dp_rank = slowfast, dp_size, dp_rank
        for _ in range(dp_rank):
            self.inner.fast_step()

    def fast_step(self) -> None:
        for _ in range(self.dp_size):
            self.inner.fast_step()

    def __next__(self):
        item = next(self.inner)
        for _ in range(self.dp_size - 1):
            self.inner.fast_step()
        return item

    def __len__(self) -> int:
        return len(self.inner) // self.dp_size

    def state_dict(self) -> dict:
        return {"inner": self.inner.state_dict(), "dp_size": self.dp_size}

    def load_state_dict(self, state: dict) -> None:
        # the saved state is the one of DP rank 0 (it points at that rank's next item)
        self.inner.load_state_dict(state["inner"])
        for _ in range(self.dp_rank):
            self.inner.fast_step()
