"""Parameter groups by weight-decay / learning-rate multipliers and free-form tags (reference
``steptronoss/optimizer/utils.py:10-72``), for code that builds a plain ``torch.optim`` optimizer; the gradient
managers of this framework read the same multipliers per parameter from the optimizer configuration."""
from __future__ import annotations

from collections.abc import Callable

from ..utils.general import convert_num
from ..utils.logger import logger


def default_wd_cond(name: str, param) -> float:
    """No weight decay on biases and one-dimensional parameters (norm gains)."""
    return 0.0 if name.endswith(".bias") or param.dim() == 1 else 1.0


def default_lr_cond(name: str, param) -> float:
    return float(getattr(param, "_lr_scale", 1.0))


def advanced_get_param_groups(module, scale_wd_cond: Callable = default_wd_cond, scale_lr_cond: Callable = default_lr_cond,
                              **special_tags) -> list:
    """One group per distinct ``(bucket prefix, wd_mult, lr_mult, tags...)``; each ``special_tags[name](param_name,
    param)`` adds a key ``name`` to the group (e.g. ``is_muon_param``).  Parameters with
    ``manual_grad_bucket_prefix`` are kept in groups of their own."""
    groups: dict = {}
    names = list(special_tags)
    for pname, p in module.named_parameters():
        if not p.requires_grad:
            continue
        key = (getattr(p, "manual_grad_bucket_prefix", None) or "default", float(scale_wd_cond(pname, p)),
               float(scale_lr_cond(pname, p)), tuple(special_tags[n](pname, p) for n in names))
        groups.setdefault(key, []).append(p)
    out = []
    for i, ((_prefix, wd, lr, tags), params) in enumerate(groups.items()):
        g = {"params": params, "wd_mult": wd, "lr_mult": lr, **dict(zip(names, tags))}
        out.append(g)
        extra = "; ".join(f"{k}: {v}" for k, v in g.items() if k != "params")
        logger.info(f"Optim group {i} -> # params: {convert_num(sum(p.numel() for p in params))}; {extra}", at=0)
    return out
