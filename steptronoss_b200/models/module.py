"""Base module with pipeline-stage structure (reference ``steptronoss/model/module.py:32-248``).

``forward = forward_head (first stage) -> forward_chunk (every stage) -> forward_tail (last
stage)``; intermediate stages receive their input through ``set_input_tensor``.  ``Float16Module``
wraps a model whose parameters are kept in bf16/fp16.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from ..parallel.layers import init_parallel_weight_, set_defaults_if_not_set_tensor_model_parallel_attributes
from ..parallel.state import PM


class MegatronModule(nn.Module):
    need_mtp_sync: bool = False
    """True on a chunk that holds a copy of the token embedding shared with another pipeline stage
    (``parallel/embedding_sync.py``); such a chunk also defines ``shared_embedding_parameters()``."""

    def __init__(self, vpp_rank: int | None = None):
        super().__init__()
        self.vpp_rank = vpp_rank if vpp_rank is not None else PM.get_vpp_rank()
        self.input_tensor = None
        self.reshaper = None  # HF <-> native weight mapping (checkpointing/reshape_ops.py)

    # ---------------------------------------------------------------- pipeline position
    @property
    def pp_rank(self) -> int:
        return self.vpp_rank * PM.size_of("PP") + PM.rank_in("PP")

    @property
    def pp_size(self) -> int:
        return PM.size_of("PP") * PM.get_vpp_size()

    @property
    def is_first_stage(self) -> bool:
        return self.pp_rank == 0

    @property
    def is_last_stage(self) -> bool:
        return self.pp_rank == self.pp_size - 1

    def set_input_tensor(self, t) -> None:
        self.input_tensor = t

    def shared_embedding_parameters(self) -> list:
        raise NotImplementedError(f"{type(self).__name__} sets need_mtp_sync but names no shared embedding parameters")

    # ---------------------------------------------------------------- forward skeleton
    def forward_head(self, **data):
        raise NotImplementedError

    def forward_chunk(self, hidden, **data):
        raise NotImplementedError

    def forward_tail(self, hidden, **data):
        raise NotImplementedError

    def forward(self, **data):
        if self.is_first_stage:
            hidden = self.forward_head(**data)
        else:
            hidden = self.input_tensor
        hidden = self.forward_chunk(hidden, **data)
        if self.is_last_stage:
            return self.forward_tail(hidden, **data)
        return hidden

    def abstract_forward(self, **data):
        """The whole model on one stage: head, chunk and tail in a row (what the pipeline split is a split of)."""
        if self.pp_size != 1:
            raise AssertionError("abstract_forward describes the unsplit model; this one is split over pipeline stages")
        return self.forward_tail(self.forward_chunk(self.forward_head(**data), **data), **data)

    # ---------------------------------------------------------------- weights
    def init_model_weight(self, seed: int = 0, std: float = 0.02) -> None:
        """``init_weights`` under the reference's name (model/module.py:142-159): afterwards every parameter carries
        ``has_initialized = True``, which the checkpoint loaders read to tell loaded from merely initialised weights."""
        self.init_weights(seed, std)
        for p in self.parameters():
            p.has_initialized = True

    def init_weights(self, seed: int = 0, std: float = 0.02) -> None:
        """Seed-deterministic N(0, std) init, independent of the parallel layout; norm weights 1 (or 0)."""
        for name, p in self.named_parameters():
            set_defaults_if_not_set_tensor_model_parallel_attributes(p)
            init_parallel_weight_(p, name, seed, std)

    def load_hf_state_dict(self, hf_state: dict, strict: bool = True) -> list:
        """Copy the HF tensors into the parameters they map to.  A tensor whose shape differs from its parameter
        (a value head in place of the LM head, a resized vocabulary) raises when ``strict``, is skipped otherwise;
        returns the names of the parameters that were skipped."""
        if self.reshaper is None:
            raise NotImplementedError(f"{type(self).__name__} has no HF reshaper")
        native = self.reshaper.forward(hf_state)
        own = dict(self.named_parameters())
        skipped = []
        for k, v in native.items():
            if k not in own:
                continue
            if tuple(own[k].shape) != tuple(v.shape):
                if strict:
                    raise RuntimeError(f"{k}: checkpoint tensor {tuple(v.shape)} does not fit parameter {tuple(own[k].shape)}")
                skipped.append(k)
                continue
            own[k].data.copy_(v.to(own[k].dtype))
            own[k].has_initialized = True
        return skipped

    def hf_state_dict(self) -> dict:
        if self.reshaper is None:
            raise NotImplementedError(f"{type(self).__name__} has no HF reshaper")
        return self.reshaper.backward({k: v.detach() for k, v in self.named_parameters()})

    def name_parameters(self) -> None:
        for n, p in self.named_parameters():
            p._log_name = n


def _cast(x, dtype):
    if torch.is_tensor(x) and x.is_floating_point():
        return x.to(dtype)
    if isinstance(x, dict):
        return {k: _cast(v, dtype) for k, v in x.items()}
    if isinstance(x, (list, tuple)):
        return type(x)(_cast(v, dtype) for v in x)
    return x


class Float16Module(nn.Module):
    """Holds a half-precision model; floating inputs are cast at the first stage and (optionally)
    outputs up-cast to fp32 at the last one."""

    def __init__(self, module: MegatronModule, params_dtype=torch.bfloat16, fp32_output: bool = True):
        super().__init__()
        self.module = module
        self.params_dtype = params_dtype
        self.fp32_output = fp32_output

    def set_input_tensor(self, t):
        return self.module.set_input_tensor(t)

    def forward(self, **data):
        if self.module.is_first_stage:
            data = {k: (v if k in ("loss_weights", "loss_masks") else _cast(v, self.params_dtype)) for k, v in data.items()}
        out = self.module(**data)
        if self.module.is_last_stage and self.fp32_output and torch.is_tensor(out):
            out = out.float()
        return out

    def state_dict(self, *a, **k):
        return self.module.state_dict(*a, **k)

    def load_state_dict(self, sd, strict=True):
        return self.module.load_state_dict(sd, strict=strict)

    def __getattr__(self, name):
        try:
            return super().__getattr__(name)
        except AttributeError:
            return getattr(self.module, name)


class ModelWrapperBase(nn.Module):
    """A wrapper that stands for the model it holds: ``forward``, ``state_dict`` and ``load_state_dict`` go to
    ``self.module`` (so checkpoints carry the inner model's keys), ``unwrap_model`` sees through it.  Base for wrappers
    of one's own (an activation logger, a precision shim); reference: model/module.py:176-191."""

    def __init__(self, module: nn.Module):
        super().__init__()
        self.module = module

    def forward(self, *inputs, **kwargs):
        return self.module(*inputs, **kwargs)

    def state_dict(self, *a, **k):
        return self.module.state_dict(*a, **k)

    def load_state_dict(self, sd, strict=True):
        return self.module.load_state_dict(sd, strict=strict)


def conversion_helper(val, conversion):
    """``conversion`` applied to ``val``, or to every leaf of nested tuples / lists (their types are kept)."""
    if isinstance(val, (tuple, list)):
        return type(val)(conversion_helper(v, conversion) for v in val)
    return conversion(val)


def fp32_to_float16(val, dtype=torch.bfloat16):
    """fp32 tensors inside ``val`` cast to ``dtype``; everything else untouched."""
    return conversion_helper(val, lambda v: v.to(dtype) if torch.is_tensor(v) and v.dtype == torch.float32 else v)


def float16_to_fp32(val):
    """bf16 / fp16 tensors inside ``val`` cast to fp32; everything else untouched."""
    return conversion_helper(val, lambda v: v.float() if torch.is_tensor(v) and v.dtype in (torch.bfloat16, torch.float16) else v)


def unwrap_model(m):
    while isinstance(m, (Float16Module, ModelWrapperBase)):
        m = m.module
    return m


def init_weight_callback(cls, init_method: str = "init_model_weight"):
    """Class decorator: after ``cls(...)`` has built an instance of exactly ``cls`` (not of a subclass, whose own
    decoration does it), call ``init_method()`` on every sub-module that has one, children before parents, and then
    on the instance (reference: model/utils/utils.py:7-25)."""
    built = cls.__init__

    def run(module):
        for child in module.children():
            run(child)
        fn = getattr(module, init_method, None)
        if callable(fn):
            fn()

    def __init__(self, *args, **kwargs):
        built(self, *args, **kwargs)
        if type(self) is cls:
            run(self)

    cls.__init__ = __init__
    return cls


def load_model_checkpoint(models, state_dict: dict, strict_load_model: bool = True) -> None:
    """Load ``state_dict["model"]`` into the model chunks of this rank: a list with one native state dict per chunk,
    or a path to HF safetensors (every chunk takes what it holds through its reshaper).  Parameters that received a
    value are marked ``has_initialized`` (reference: model/utils/utils.py:28-65)."""
    from ..utils.logger import logger

    if "model" not in state_dict:
        raise AssertionError("state_dict must contain 'model' key.")
    source = state_dict["model"]
    if isinstance(source, str):
        from ..utils.weight_loader import HFWeights

        source = state_dict["model"] = HFWeights(source)
        from_hf = True
    else:
        from_hf = False
    for vid, model in enumerate(models):
        model = unwrap_model(model)
        PM.set_vpp_rank(vid)
        if from_hf:
            skipped = set(model.load_hf_state_dict(source, strict=strict_load_model))
            if skipped:
                logger.warning(f"model chunk {vid}: not loaded (shape differs): {sorted(skipped)}", at=None)
            continue                                      # load_hf_state_dict marks what it copied
        msg = model.load_state_dict(source[vid], strict=strict_load_model)
        missing = set(msg.missing_keys)
        if missing or msg.unexpected_keys:
            logger.warning(f"model chunk {vid}: {msg}", at=None)
        for name, p in model.named_parameters():
            if name not in missing:
                p.has_initialized = True
