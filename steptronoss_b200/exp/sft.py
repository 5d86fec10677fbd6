"""Supervised fine-tuning experiment and its packed-chat data configuration.

Reference: ``steptronoss/exp/sft.py:22-49`` (node set) and the packing / batch contract of
``playground/data/sft/oss260312/step_sft_data_config0311.py:207-286``.

A packed micro-batch is built from the samples of one packed sequence: for every sample the inputs are
``tokens[:-1]``, the labels ``tokens[1:]`` and the loss mask ``loss_mask[1:]`` (shift by one *per document*,
so no position predicts across a document border); the documents are concatenated, a dummy masked-out
document pads the total to a multiple of ``seqlen_divisible_by`` (tensor-/sequence-parallel alignment), and
``cu_seqlens`` (int32), ``max_seq_len`` and per-document ``position_id`` describe the layout.
"""
from __future__ import annotations

import numpy as np
import torch

from ..config import Config, Ref
from ..models.decoder_model import DecoderLLMConfig
from .base_exp import BaseExp, DataConfig, GradientManagerConfig, ProfilerConfig
from .checkpointing import CheckpointConfig
from .lr_schedulers import SchedulerConfig
from .ntp import NTPTrainerConfig, PretrainMetricConfig


class SFTDatasetsConfig(Config):
    def build_datasets(self) -> dict:
        """``{domain: (dataset, epochs)}``; every sample is ``{"tokens": [...], "loss_mask": [...]}``."""
        raise NotImplementedError


class SFTDataConfig(DataConfig):
    dataset_cfg: SFTDatasetsConfig = SFTDatasetsConfig
    oversize_policy: str = "drop"
    max_packing_seqlen = Ref("..trainer_cfg.global_seq_length", 8192)
    seqlen_divisible_by: int = 64
    global_data_keys = ["cu_seqlens", "position_id"]
    dataset_sampling: str = "sequential"
    num_workers: int = 16
    pin_memory: bool = True

    def build_dataloader(self, dp_rank: int = 0, dp_size: int = 1):
        from ..data.async_accelerate import async_accelerate_slowfast
        from ..data.dataloader import MixedPackedDataloader
        from ..data.nextable import DPMux

        datasets = self.dataset_cfg.build_datasets()
        dl = MixedPackedDataloader([d for d, _ in datasets.values()], [e for _, e in datasets.values()],
                                   max_length=self.max_packing_seqlen, oversize_policy=self.oversize_policy,
                                   transform=self.pack, dataset_sampling=self.dataset_sampling)
        dl = DPMux(dl, dp_size=dp_size, dp_rank=dp_rank)
        if self.num_workers > 0:
            dl = async_accelerate_slowfast(dl, num_workers=self.num_workers, pin_memory=self.pin_memory)
        return dl

    def pack(self, pieces: list) -> dict:
        from ..utils.general import get_position_id_from_cu_seqlens

        pieces = list(pieces)
        size = sum(len(s["tokens"]) - 1 for s in pieces)
        rem = size % self.seqlen_divisible_by
        if rem:
            pad = np.zeros(self.seqlen_divisible_by - rem + 1, dtype=np.int64)
            pieces.append({"tokens": pad, "loss_mask": pad})
        sizes = torch.tensor([len(s["tokens"]) - 1 for s in pieces])
        as_t = lambda x, dt: torch.as_tensor(np.asarray(x), dtype=dt)  # noqa: E731
        tokens = torch.cat([as_t(s["tokens"][:-1], torch.long) for s in pieces])
        labels = torch.cat([as_t(s["tokens"][1:], torch.long) for s in pieces])
        loss_mask = torch.cat([as_t(s["loss_mask"][1:], torch.float32) for s in pieces])
        cu = torch.cat([torch.zeros(1, dtype=torch.int64), torch.cumsum(sizes, 0)]).int()
        return dict(tokens=tokens, labels=labels, loss_mask=loss_mask, cu_seqlens=cu, max_seq_len=sizes.max(),
                    position_id=get_position_id_from_cu_seqlens(cu))

    def preprocess(self, batch: dict) -> dict:
        dev = "cuda" if torch.cuda.is_available() else "cpu"
        cu = batch["cu_seqlens"].to(dev, non_blocking=True)
        out = dict(cu_seqlens=cu, max_seq_len=int((batch["cu_seqlens"][1:] - batch["cu_seqlens"][:-1]).max()),
                   position_id=batch["position_id"].to(dev, non_blocking=True))
        if "tokens" in batch:  # first / last pipeline stage
            out.update(input_ids=batch["tokens"].to(dev, non_blocking=True)[None],
                       labels=batch["labels"].to(dev, non_blocking=True)[None],
                       loss_masks=batch["loss_mask"].to(dev, non_blocking=True)[None])
        return out


class SFTExp(BaseExp):
    trainer_cfg: NTPTrainerConfig = NTPTrainerConfig
    model_cfg: DecoderLLMConfig = DecoderLLMConfig
    optimizer_cfg: GradientManagerConfig = GradientManagerConfig
    scheduler_cfg: SchedulerConfig = SchedulerConfig
    data_cfg: SFTDataConfig = SFTDataConfig
    checkpoint_cfg: CheckpointConfig = CheckpointConfig
    metric_cfg: PretrainMetricConfig = PretrainMetricConfig
    profiler_cfg: ProfilerConfig = ProfilerConfig

    def train(self):
        self.update_from_args()
        self.sanity_check()
        trainer = self.trainer_cfg.get_trainer_cls()(exp=self)
        self.configure_optimizable()
        trainer.train()
        return trainer

    def configure_optimizable(self) -> None:
        """Hook between building the trainer and training: an experiment selects operator back-ends here with
        ``utils.optimizable.set_optimization`` (the reference's experiment files do; its names are understood)."""
