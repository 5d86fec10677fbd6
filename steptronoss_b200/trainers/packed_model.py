"""Model + gradient manager + LR scheduler as one unit, with host offload of each part.

Reference: ``steptronoss/core/trainers/packed_model.py:23-305``.  RL jobs keep several of these in one
process (policy, reference policy, critic ...) and swap them in and out of device memory around each phase.
With bf16 parameters, an fp32 gradient buffer and fp32 masters + two Adam moments a model of N parameters
holds ``2N + 4N + 12N/DP`` bytes on the device; the three parts are offloaded independently:

* parameters: the flat bf16 buffers move to pinned host memory and the parameters are re-seated as views
  of the host copy (one copy per bucket, not one per tensor);
* gradient buffers: freed and re-created zeroed;
* optimizer state: the flat fp32 shards move to the host.

State dicts are passed at construction so that the model, optimizer and scheduler are hydrated before any
flat buffer or hook exists.
"""
from __future__ import annotations

from contextlib import contextmanager, nullcontext

import torch

from ..models.module import Float16Module, unwrap_model
from ..parallel.state import PM
from ..utils.dist_utils import broadcast_tensors
from ..utils.dev_utils import print_n_params
from ..utils.logger import logger
from ..utils.timers import get_timers


def moving_iter(items: list):
    """Iterate over ``items`` moving each element to the current device just before it is used."""
    from ..utils.general import recur_to

    dev = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
    for it in items:
        yield recur_to(it, dev)


class PackedModel:
    def __init__(self, trainer_config, model_config, grad_manager_config=None, scheduler_config=None,
                 training: bool = False, state_dicts: dict | None = None, strict_load_model: bool = False,
                 name: str = "packed_model", seed: int = 0):
        state_dicts = state_dicts or {}
        self.name, self.training = name, training
        self.model_config, self.trainer_config, self.scheduler_config = model_config, trainer_config, scheduler_config
        self.seed = seed
        self.models = self.setup_model(model_config)
        if "model" in state_dicts:
            self._load_model_state(state_dicts, strict_load_model)
        self._offloaded = {"params": False, "grad_buffer": False, "optimizer_state": False}
        self.grad_manager = self.scheduler = None
        if training:
            self.grad_manager = grad_manager_config.build_gradient_manager(self.models)
            if "optimizer" in state_dicts:
                self.grad_manager.load_state_dict(state_dicts["optimizer"])
            elif "model" in state_dicts:
                self.grad_manager.refresh_masters_from_params()
            self.scheduler = scheduler_config.build_scheduler(self.grad_manager.optimizer)
            if "scheduler" in state_dicts:
                self.scheduler.load_state_dict(state_dicts["scheduler"])

    # ------------------------------------------------------------------ construction
    def setup_model(self, model_config) -> torch.nn.ModuleList:
        dev = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
        self.device = dev
        chunks = []
        for vp in range(PM.get_vpp_size()):
            PM.set_vpp_rank(vp)
            with torch.device(dev):
                m = model_config.build_model(vpp_rank=vp) if PM.get_vpp_size() > 1 else model_config.build_model()
            m.init_weights(self.seed, getattr(model_config, "init_std", 0.02))
            chunks.append(Float16Module(m, model_config.params_dtype, getattr(model_config, "fp32_output", True)))
        PM.set_vpp_rank(0)
        print_n_params(chunks)
        return torch.nn.ModuleList(chunks)

    def _load_model_state(self, state_dicts: dict, strict: bool) -> None:
        for i, m in enumerate(self.models):
            key = "model" if i == 0 else f"model{i}"
            if key in state_dicts:
                unwrap_model(m).load_state_dict(state_dicts[key], strict=strict)

    # ------------------------------------------------------------------ offload
    def _params_to(self, device, non_blocking: bool) -> None:
        # modules without a gradient manager own plain tensors: move them one by one
        for m in self.models:
            for p in m.parameters():
                p.data = p.data.to(device, non_blocking=non_blocking)
            for b in m.buffers():
                b.data = b.data.to(device, non_blocking=non_blocking)

    def _offload_param(self, non_blocking: bool = True) -> None:
        if self._offloaded["params"]:
            return
        self._offloaded["params"] = True
        if self.grad_manager is not None:
            self.grad_manager.offload_params(non_blocking)
        else:
            self._params_to("cpu", non_blocking)

    def _backload_param(self, non_blocking: bool = True) -> None:
        if not self._offloaded["params"]:
            return
        self._offloaded["params"] = False
        if self.grad_manager is not None:
            self.grad_manager.reload_params(non_blocking)
        else:
            self._params_to(self.device, non_blocking)

    def _offload_grad_buffer(self) -> None:
        """Also discards the accumulated gradients."""
        if self._offloaded["grad_buffer"] or not self.training:
            return
        self._offloaded["grad_buffer"] = True
        self.grad_manager.destroy_buffer()

    def _backload_grad_buffer(self) -> None:
        if not self._offloaded["grad_buffer"] or not self.training:
            return
        self._offloaded["grad_buffer"] = False
        self.grad_manager.build_buffer()

    def _offload_optimizer_state(self) -> None:
        if self._offloaded["optimizer_state"]:
            return
        self._offloaded["optimizer_state"] = True
        if not self.training:
            logger.warning("no optimizer state needs offload")
            return
        self.grad_manager.offload_state()

    def _backload_optimizer_state(self) -> None:
        if not self._offloaded["optimizer_state"]:
            return
        self._offloaded["optimizer_state"] = False
        if not self.training:
            logger.warning("no optimizer state needs backload")
            return
        self.grad_manager.reload_state()

    def offload_model(self) -> None:
        with get_timers().record(f"{self.name}_offload_model", 1):
            self._offload_param(True)

    def backload_model(self) -> None:
        with get_timers().record(f"{self.name}_backload_model", 1):
            self._backload_param(True)

    def offload_state(self) -> None:
        if self.training:
            with get_timers().record(f"{self.name}_offload_state", 1):
                self._offload_grad_buffer()
                self._offload_optimizer_state()

    def backload_state(self) -> None:
        if self.training:
            with get_timers().record(f"{self.name}_backload_state", 1):
                self._backload_grad_buffer()
                self._backload_optimizer_state()

    @contextmanager
    def on_gpu(self, model: bool = True, optimizer: bool = True):
        if model:
            self.backload_model()
        if optimizer:
            self.backload_state()
        try:
            yield
        finally:
            if model:
                self.offload_model()
            if optimizer:
                self.offload_state()

    # ------------------------------------------------------------------ stepping
    def optimizer_step(self):
        assert self.training
        ok, grad_norm, zeros = self.grad_manager.step()
        tc, sc = self.trainer_config, self.scheduler_config
        unit = getattr(sc, "scheduler_unit", "iter")
        inc = {"iter": 1, "sample": tc.global_batch_size,
               "token": tc.global_batch_size * tc.global_seq_length}[unit]
        self.scheduler.step(inc)
        for m in self.models:
            um = unwrap_model(m)
            if hasattr(um, "after_optimizer_step"):
                um.after_optimizer_step()
        if getattr(tc, "empty_unused_memory_level", 0) >= 2 and torch.cuda.is_available():
            torch.cuda.empty_cache()
        return ok, grad_norm, zeros

    def build_vpp_iterators(self, builder) -> list:
        its = []
        for vp in range(PM.get_vpp_size()):
            PM.set_vpp_rank(vp)
            its.append(builder() if self.trainer_config.is_data_source() else None)
        PM.set_vpp_rank(0)
        return its

    def forward_backward(self, data_list: list, data_proc_fn, loss_fn=None, training: bool | None = None,
                         zero_grad: bool = True, offload_opt_while_forward: bool = False,
                         collect_output: bool = False, offload_data: bool = False) -> list:
        """Run the micro-batch schedule over ``data_list`` (needed on the data-source ranks only).

        ``data_proc_fn(data) -> kwargs of the model``; ``loss_fn(data, output, loss_scale)``; returns the
        collected last-stage outputs when ``collect_output``."""
        training = self.training if training is None else training
        if training:
            if zero_grad:
                self.grad_manager.zero_grad()
            self.grad_manager.wait_param_gather()
            if offload_opt_while_forward:
                self._offload_optimizer_state()
        n = len(data_list) if data_list else None
        if PM.size_of("MP") > 1:
            n = broadcast_tensors(n, src=PM.ranks_of("MP")[0], group=PM.group_of("MP"))
        its = self.build_vpp_iterators((lambda: moving_iter(data_list)) if offload_data else (lambda: iter(data_list)))
        with nullcontext() if training else torch.no_grad():
            sched = self.model_config.get_pp_scheduler()
            sched.configure(self.models, its, data_sync_fn=self.trainer_config.sync_get_data, loss_fn=loss_fn,
                            data_proc_fn=data_proc_fn, training=training, collect_output=collect_output)
            outputs = sched.run(n)
        if training and offload_opt_while_forward:
            self._backload_optimizer_state()
        return outputs

    def state_dicts(self) -> dict:
        out = {("model" if i == 0 else f"model{i}"): unwrap_model(m).state_dict() for i, m in enumerate(self.models)}
        if self.training:
            out["optimizer"] = self.grad_manager.state_dict()
            out["scheduler"] = self.scheduler.state_dict()
        return out
