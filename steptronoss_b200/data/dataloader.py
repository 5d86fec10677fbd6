"""Resumable data loaders (reference ``steptronoss/data/dataloader/{base_dataloader,packed_dataloader}.py``).

``BaseDataloader``: a dataset indexed by a sampler.  ``MixedPackedDataloader``: a weighted mixture of datasets
whose whole sampling order is drawn up front (weight of a dataset = epochs x size), greedily packed into
sequences of at most ``max_length`` tokens without truncation; item ``i`` is the list of samples of packed
sequence ``i`` (optionally passed through ``transform``, typically the batch builder).  The only state is the
index of the next packed sequence.
"""
from __future__ import annotations

from collections.abc import Callable
from typing import Any

from ..utils.logger import logger
from .nextable import LazyUpdateNextable
from .packing import PackingResult, pack
from .samplers import LoopedSequentialSampler, LoopedShuffleSampler, WeightedRandomSampler


class BaseDataloader(LazyUpdateNextable):
    def __init__(self, dataset, sampler) -> None:
        if not hasattr(sampler, "get") or not hasattr(sampler, "update"):
            raise TypeError("sampler must implement get() and update()")
        self.dataset, self.sampler = dataset, sampler

    def __len__(self) -> int:
        return len(self.dataset)

    def get(self) -> Any:
        return self.dataset[self.sampler.get()]

    def update(self) -> None:
        self.sampler.update()

    def state_dict(self) -> dict:
        return {"sampler": self.sampler.state_dict()} if hasattr(self.sampler, "state_dict") else {}

    def load_state_dict(self, state: dict) -> None:
        if state.get("sampler") is not None and hasattr(self.sampler, "load_state_dict"):
            self.sampler.load_state_dict(state["sampler"])


class MixedPackedDataloader(LazyUpdateNextable):
    def __init__(self, datasets: list, epochs: list, max_length: int, oversize_policy: str = "extend",
                 transform: Callable | None = None, dataset_sampling: str | list = "random"):
        if not datasets:
            raise ValueError("datasets cannot be empty.")
        if len(datasets) != len(epochs):
            raise ValueError("datasets and epochs must have the same length.")
        if isinstance(dataset_sampling, str):
            dataset_sampling = [dataset_sampling] * len(datasets)
        if len(dataset_sampling) != len(datasets):
            raise ValueError("dataset_sampling list must have the same length as datasets.")
        bad = [s for s in dataset_sampling if s not in ("sequential", "random")]
        if bad:
            raise ValueError(f"dataset_sampling contains unsupported strategy: {bad[0]!r}. "
                             "Supported strategies are 'sequential' and 'random'.")
        self.datasets, self.ds_epochs, self.transform = datasets, epochs, transform
        self.dataset_sampling = list(dataset_sampling)
        self.piece_order, self.packing_result = self._schedule_all(max_length, oversize_policy)
        self._pack_ranges = self.packing_result.packed_sample_ranges
        if not self._pack_ranges:
            raise ValueError("packed dataset is empty.")
        self.data_idx = 0

    @staticmethod
    def _sample_sizes(ds) -> list:
        meta = getattr(ds, "sample_meta", None)
        if meta and isinstance(meta[0], int) and meta[0] == len(ds[0]["tokens"]):
            return list(meta)
        logger.warning("Measuring every sample of a dataset; compile it with the token count as sample meta "
                       "to avoid this pass.")
        return [len(x["tokens"]) if isinstance(x, dict) and "tokens" in x else len(x) for x in ds]

    def _schedule_all(self, max_length: int, oversize_policy: str) -> tuple[list, PackingResult]:
        sizes, inner, weights = [], [], []
        for i, (ds, ep, how) in enumerate(zip(self.datasets, self.ds_epochs, self.dataset_sampling)):
            n = len(ds)
            if n <= 0:
                raise ValueError("Dataset is empty.")
            if float(ep) <= 0:
                raise ValueError("Epoch must be positive.")
            sizes.append(self._sample_sizes(ds))
            inner.append(LoopedShuffleSampler(n, seed=1234 + i) if how == "random" else LoopedSequentialSampler(n))
            weights.append(float(ep) * n)
        outer = WeightedRandomSampler(weights)
        order, piece_sizes = [], []
        for _ in range(int(sum(weights))):
            d = next(outer)
            j = next(inner[d])
            order.append((d, j))
            piece_sizes.append(sizes[d][j])
        result = pack(piece_sizes, max_len=max_length, oversize_policy=oversize_policy)
        if result.num_droped:
            logger.warning(f"{result.num_droped} sample droped for oversize!")
        return order, result

    def __len__(self) -> int:
        return len(self._pack_ranges)

    def get(self) -> Any:
        start, count = self._pack_ranges[self.data_idx % len(self._pack_ranges)]
        items = [self.datasets[d][j] for d, j in self.piece_order[start:start + count]]
        return self.transform(items) if self.transform else items

    def update(self) -> None:
        self.data_idx += 1

    def state_dict(self) -> dict:
        return {"data_idx": self.data_idx}

    def load_state_dict(self, state: dict) -> None:
        self.data_idx = state.get("data_idx", self.data_idx)
