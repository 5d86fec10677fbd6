"""Optimizer configuration (reference ``steptronoss/exp/optimizer.py:12-195``)."""
from __future__ import annotations

import torch

from ..config import Ref
from .abstract import OptimizerConfig as AbstractOptimizerConfig


class OptimizerConfig(AbstractOptimizerConfig):
    weight_decay: float
    weight_decay_on_1d_params: bool
    lr: float
    is_muon = False

    def scale_lr_func(self, name: str, param) -> float:
        return float(getattr(param, "_lr_scale", 1.0))

    def scale_wd_cond(self, name: str, param) -> float:
        if name.endswith(".bias") or (param.dim() == 1 and not self.weight_decay_on_1d_params):
            return 0.0
        return 1.0

    def build_optimizer(self, model):
        """The optimizer state lives inside the gradient manager (flat shards); this returns the
        plain-PyTorch equivalent for code that wants a standalone ``torch.optim`` object."""
        raise NotImplementedError


class AdamConfig(OptimizerConfig):
    lr: float = Ref("...scheduler_cfg.lr", 1e-4)
    weight_decay: float = Ref("...scheduler_cfg.weight_decay", 0.0)
    weight_decay_on_1d_params: bool = False
    adam_eps: float = 1e-8
    adam_beta1: float = 0.9
    adam_beta2: float = 0.95

    def param_groups(self, model):
        groups: dict = {}
        for name, p in model.named_parameters():
            if not p.requires_grad:
                continue
            key = (self.scale_lr_func(name, p), self.scale_wd_cond(name, p))
            groups.setdefault(key, []).append(p)
        return [{"params": ps, "lr": self.lr * k[0], "weight_decay": self.weight_decay * k[1], "lr_mult": k[0],
                 "wd_mult": k[1]} for k, ps in groups.items()]

    def build_optimizer(self, model):
        return torch.optim.Adam(self.param_groups(model), lr=self.lr, weight_decay=self.weight_decay,
                                betas=(self.adam_beta1, self.adam_beta2), eps=self.adam_eps)


class MuonConfig(OptimizerConfig):
    """Muon for the 2-D hidden matrices, AdamW for everything else."""

    lr: float = Ref("...scheduler_cfg.lr", 1e-4)
    weight_decay: float = Ref("...scheduler_cfg.weight_decay", 0.0)
    weight_decay_on_1d_params: bool = False
    is_muon = True
    muon_momentum: float = 0.95
    muon_nesterov: bool = True
    muon_matched_adamw_rms: float = 0.2
    muon_ns_steps: int = 5
    muon_run_ns_in_fp16: bool = True
    muon_newtonschulz_fn: str = "default"
    adam_eps: float = 1e-8
    adam_beta1: float = 0.9
    adam_beta2: float = 0.95
    muon_param_attr_only: bool = False
    muon_exclude_embeddings: bool = True
    muon_exclude_names: tuple = ()
    muon_min_ndim_is_2_only: bool = True
    """True: only ``ndim == 2`` parameters; False: ``ndim >= 2`` (stacked expert weights, one
    Newton-Schulz per expert matrix; reference ``playground/sft/step3/muon_optimizer.py``)."""

    def mark_muon_params(self, model) -> None:
        exclude = tuple(self.muon_exclude_names or ())
        emb = set()
        if self.muon_exclude_embeddings:
            for mod in model.modules():
                if isinstance(mod, torch.nn.Embedding) or "Embedding" in type(mod).__name__:
                    for w in mod.parameters(recurse=True):
                        emb.add(id(w))
        for name, p in model.named_parameters():
            if getattr(p, "is_muon_param", False) is True and hasattr(p, "_muon_explicit"):
                continue
            if self.muon_param_attr_only or id(p) in emb or any(t in name for t in exclude):
                flag = bool(getattr(p, "_muon_explicit", False))
            else:
                flag = p.dim() == 2 if self.muon_min_ndim_is_2_only else p.dim() >= 2
            p.is_muon_param = flag

    def mark_gather_ops(self, model) -> None:
        """Attach ``merge_op`` (how to rebuild the full matrix from TP shards) to every parameter."""
        from ..checkpointing.reshape_ops import merge_op_for

        for _, p in model.named_parameters():
            if p.requires_grad:
                p.merge_op = merge_op_for(p)

    def build_optimizer(self, model):
        from ..optim.muon import Muon

        self.mark_muon_params(model)
        muon, other = [], []
        for n, p in model.named_parameters():
            if p.requires_grad:
                (muon if p.is_muon_param else other).append(p)
        groups = [{"params": muon, "is_muon_param": True}, {"params": other, "is_muon_param": False}]
        return Muon(groups, lr=self.lr, weight_decay=self.weight_decay, matched_adamw_rms=self.muon_matched_adamw_rms,
                    momentum=self.muon_momentum, nesterov=self.muon_nesterov, ns_steps=self.muon_ns_steps,
                    adamw_betas=(self.adam_beta1, self.adam_beta2), adamw_eps=self.adam_eps,
                    run_ns_in_fp16=self.muon_run_ns_in_fp16, newtonschulz_fn=self.muon_newtonschulz_fn)
