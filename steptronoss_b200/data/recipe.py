"""Declarative description of SFT / RL training data (reference ``steptronoss/data/recipe.py:14-123``):
named domains made of source files with optional sub-sampling, and how many epochs of each domain go into
the mixture."""
from __future__ import annotations

from dataclasses import dataclass


@dataclass
class DataSourceFile:
    path: str
    subsample_rate: float = 1.0

    def __post_init__(self):
        if not self.path:
            raise ValueError("DataSourceFile 'path' cannot be empty.")
        if not 0.0 < self.subsample_rate <= 1.0:
            raise ValueError(f"DataSourceFile 'subsample_rate' must be in (0.0, 1.0]. Got: {self.subsample_rate} "
                             f"for file '{self.path}'")


def _check_epochs(domains: dict, epochs: dict) -> None:
    if not domains:
        raise ValueError("'domains' cannot be empty.")
    if not epochs:
        raise ValueError("'epochs' cannot be empty.")
    unknown = set(epochs) - set(domains)
    if unknown:
        raise ValueError(f"Domain(s) {sorted(unknown)} from 'epochs' are not defined in 'domains'.")
    missing = set(domains) - set(epochs)
    if missing:
        raise ValueError(f"Data domain(s) {sorted(missing)} are missing a corresponding configuration in 'epochs'.")
    for name, e in epochs.items():
        if e <= 0.0:
            raise ValueError(f"Epochs for domain '{name}' must be positive. Got: {e}")


@dataclass(eq=False)
class DataRecipe:
    domains: dict
    """domain name -> list of :class:`DataSourceFile`"""
    epochs: dict
    """domain name -> epochs of that domain in the mixture"""

    def __post_init__(self):
        _check_epochs(self.domains, self.epochs)

    def to_dict(self, rep: bool = False) -> dict:
        return {"domains": self.domains, "epochs": self.epochs}

    def __eq__(self, other):
        return isinstance(other, DataRecipe) and self.domains == other.domains and self.epochs == other.epochs


@dataclass(eq=False)
class CompiledDataRecipe:
    domains: dict
    """domain name -> directory of the compiled (tokenised, indexed) dataset"""
    epochs: dict

    def __post_init__(self):
        _check_epochs(self.domains, self.epochs)

    def to_dict(self, rep: bool = False) -> dict:
        return {"domains": self.domains, "epochs": self.epochs}

    def __eq__(self, other):
        return isinstance(other, CompiledDataRecipe) and self.domains == other.domains and self.epochs == other.epochs
