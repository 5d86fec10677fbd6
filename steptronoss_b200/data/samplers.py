"""Index samplers (reference ``steptronoss/data/samplers/base_sampler.py:9-170``): looped sequential,
looped shuffle (a fresh permutation per epoch from ``seed + epoch``) and a deterministic weighted sampler that
always serves the source whose served/weight ratio is lowest."""
from __future__ import annotations

import numpy as np

from .nextable import LazyUpdateNextable


class BaseSampler(LazyUpdateNextable):
    """What a sampler is: a resumable stream of indices into ``size`` items (``next(sampler) -> int``); a sampler of
    one's own subclasses this and gives ``get`` / ``update`` / ``state_dict`` / ``load_state_dict``."""

    size: int


class LoopedSequentialSampler(BaseSampler):
    def __init__(self, size: int):
        self.size, self.idx = size, 0

    def get(self) -> int:
        return self.idx % self.size

    def update(self) -> None:
        self.idx += 1

    def state_dict(self) -> dict:
        return {"idx": self.idx}

    def load_state_dict(self, state: dict) -> None:
        self.idx = state["idx"]


class LoopedShuffleSampler(BaseSampler):
    def __init__(self, size: int, seed: int = 0):
        self.size, self.seed, self.idx = size, seed, 0
        self._epoch, self._perm = -1, None

    def _permutation(self, epoch: int):
        if epoch != self._epoch:
            self._perm = np.random.default_rng([self.seed, epoch]).permutation(self.size)
            self._epoch = epoch
        return self._perm

    def get(self) -> int:
        epoch, pos = divmod(self.idx, self.size)
        return int(self._permutation(epoch)[pos])

    def update(self) -> None:
        self.idx += 1

    def state_dict(self) -> dict:
        return {"idx": self.idx, "seed": self.seed}

    def load_state_dict(self, state: dict) -> None:
        self.idx, self.seed = state["idx"], state.get("seed", self.seed)
        self._epoch = -1


class WeightedRandomSampler(BaseSampler):
    """Chooses among ``len(weights)`` sources so that the served counts follow the weights: the next source
    is ``argmin((served + 1) / weight)`` (ties to the lower index) — deterministic and resumable."""

    def __init__(self, weights: list[float]):
        w = np.asarray(weights, dtype=np.float64)
        if (w <= 0).any():
            raise ValueError("weights must be positive")
        self.weights = w / w.sum()
        self.served = np.zeros(len(w), dtype=np.int64)

    def _select(self) -> int:
        return int(np.argmin((self.served + 1) / self.weights))

    def get(self) -> int:
        return self._select()

    def update(self) -> None:
        self.served[self._select()] += 1

    def state_dict(self) -> dict:
        return {"served": self.served.tolist()}

    def load_state_dict(self, state: dict) -> None:
        self.served = np.asarray(state["served"], dtype=np.int64)
