"""Next-token-prediction training: trainer config with the loss function, default metrics and the
pre-training experiment skeleton (reference ``steptronoss/exp/ntp.py:20-177``)."""
from __future__ import annotations

import os

import torch

from ..parallel.state import PM
from ..utils.metrics import GlobalMetrics
from .base_exp import BaseExp, MetricConfig, TrainerConfig


class PretrainMetricConfig(MetricConfig):
    def __init__(self) -> None:
        super().__init__()
        from ..utils.metrics import HistogramMetric, Metric, ModelLayerMetric, PercentageMetric

        self.lm_loss = Metric().mean("time").mean("dp")
        self.grad_norm = Metric().mean("time")
        self.grad_zeros = Metric().mean("time")
        self.acc = PercentageMetric().sum("time").sum("dp")
        self.logits_max = Metric().max("time").max("dp")
        self.losses = HistogramMetric()
        self.losses.enabled = False


class MoEPretrainMetricConfig(PretrainMetricConfig):
    def __init__(self) -> None:
        super().__init__()
        from ..utils.metrics import ModelLayerMetric

        for name in ("moe_aux_loss", "moe_minp", "moe_sumk", "moe_std", "moe_max", "moe_avg", "expert_coef",
                     "peak_to_avg_ratio", "router_logits_max", "router_logits_std", "zloss"):
            setattr(self, name, ModelLayerMetric().mean("time").mean("dp").sum("pp"))


MoePretrainMetricConfig = MoEPretrainMetricConfig        # the reference's spelling (exp/ntp.py)


class NTPTrainerConfig(TrainerConfig):
    micro_batch_size: int = 1
    global_batch_size: int = 8
    global_seq_length: int = 8192

    def get_trainer_cls(self):
        from ..trainers.lm_trainer import DecoderPretrainTrainer

        return DecoderPretrainTrainer

    def apply_loss_mask(self, losses: torch.Tensor, loss_mask: torch.Tensor) -> torch.Tensor:
        """Masked mean over the *global* mask count; under context parallelism the local sum is
        multiplied by CP because the DP average that follows also runs over the CP ranks."""
        cp = PM.size_of("CP")
        mask = loss_mask
        if cp > 1:
            from ..parallel.context_parallel import scatter_to_balanced_cp_region

            mask = scatter_to_balanced_cp_region(loss_mask.reshape(-1), dim=0)
        mask = mask.reshape(-1).float()
        losses = losses.reshape(-1)
        losses = torch.where(mask == 0, torch.zeros_like(losses), losses)
        denom = loss_mask.sum().clamp_min(1e-8)
        return (losses * mask).sum() / denom * cp

    def loss_func(self, data: dict, output, loss_scale: float = 1.0) -> torch.Tensor:
        """Model output -> one scalar to call ``backward()`` on (already multiplied by ``loss_scale``)."""
        if isinstance(output, dict) and "loss" in output:
            loss = output["loss"]
            with torch.no_grad():
                w = output["weights"]
                hit = ((output["pred"] == output["labels"]) & (w > 0)).sum()
                GlobalMetrics.lm_loss.add(loss.detach() / max(loss_scale, 1e-30))
                GlobalMetrics.acc.add(hit, (w > 0).sum())
                GlobalMetrics.consumed_tokens.add(float(output["labels"].numel() * PM.size_of("CP")))
            return loss
        logits = output
        if torch.is_tensor(logits) and logits.numel() == 1:
            return logits * loss_scale
        from ..ops import vocab_parallel_cross_entropy

        if data.get("loss_masks") is None and "loss_mask" in data:
            raise RuntimeError("Critical Typo: please use 'loss_masks' instead of 'loss_mask' in data!")
        labels = data["labels"].reshape(-1)
        if PM.size_of("CP") > 1:
            from ..parallel.context_parallel import scatter_to_balanced_cp_region

            labels = scatter_to_balanced_cp_region(labels, dim=0)
        tp = PM.size_of("TP")
        vstart = PM.rank_in("TP") * logits.shape[-1] if tp > 1 else 0
        losses, pred = vocab_parallel_cross_entropy(logits.float().reshape(labels.numel(), -1), labels, vstart,
                                                    PM.group_of("TP") if tp > 1 else None)
        masks = data.get("loss_masks")
        loss = self.apply_loss_mask(losses, masks) if masks is not None else losses.mean()
        GlobalMetrics.lm_loss.add(loss.detach())
        GlobalMetrics.acc.add((pred == labels).sum(), labels.numel())
        GlobalMetrics.consumed_tokens.add(float(labels.numel() * PM.size_of("CP")))
        return loss * loss_scale

    def make_logs(self, iteration, metrics, tb_writer=None):
        logs = super().make_logs(iteration, metrics, tb_writer)
        if "lm_loss" in metrics:
            logs["lm_loss"] = f"{float(metrics['lm_loss']):.6E}"
        return logs

    def sanity_check(self):
        super().sanity_check()
        assert self.global_batch_size > 0


class PretrainExp(BaseExp):
    """Experiment with the nodes a pre-training / SFT run needs: ``trainer_cfg, model_cfg,
    optimizer_cfg, scheduler_cfg, data_cfg, checkpoint_cfg, metric_cfg, profiler_cfg``."""

    def sanity_check(self):
        super().sanity_check()
        # inside a launched job the world is known; before launch (cfshow, script generation) the job the
        # resource configuration asks for is what the layout has to fit
        world = os.getenv("WORLD_SIZE")
        if world is None:
            rc = getattr(self, "resource_cfg", None)
            world = max(int(getattr(rc, "gpu", 0) or 0) * int(getattr(rc, "replica", 1) or 1), 1) if rc is not None else 1
        world = int(world)
        pc = self.model_cfg.parallel_cfg
        mp = pc.pipeline_model_parallel_size * pc.tensor_model_parallel_size * pc.context_parallel_size
        assert world >= mp and world % mp == 0, f"world {world} incompatible with PP*TP*CP = {mp}"

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
