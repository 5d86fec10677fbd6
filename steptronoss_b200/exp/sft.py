"""Supervised fine-tuning experiment (same node set as pre-training; data is packed chat samples)."""
from __future__ import annotations

from .ntp import PretrainExp


class SFTExp(PretrainExp):
    pass
