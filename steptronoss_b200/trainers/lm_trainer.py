"""SFT / pre-training loop (reference ``steptronoss/core/trainers/lm_trainer.py:37-476``).

``train_step``: zero the flat gradient buffers, run the micro-batch schedule (forward + backward
with gradients accumulated in ``main_grad``), then the gradient manager's fused reduce / clip /
Adam / parameter refresh.  Nothing in the step reads a device value on the host; the loss, the
gradient norm and the kernel status word are read only when a log line is due.
"""
from __future__ import annotations

import os
import time

import torch

from ..models.module import Float16Module, unwrap_model
from ..ops import native
from ..parallel.state import PM, set_mpu_random_seed
from ..utils.dev_utils import raise_if_nonfinite
from ..utils.logger import logger
from ..utils.memory_tracker import CMT
from ..utils.metrics import GlobalMetrics
from ..utils.timers import get_timers, init_timers
from .base_trainer import BaseTrainer


class DecoderPretrainTrainer(BaseTrainer):
    def __init__(self, exp):
        super().__init__(exp)
        self.models = []
        self.grad_manager = None
        self.scheduler = None
        self.dataloader = None
        self.data_iterators = []
        self.checkpointer = None
        self.writer = None
        self.train_iters = None
        self.history: list = []
        self.last_metrics: dict = {}
        self.consumed_samples = 0
        self._t_last = time.perf_counter()

    # ------------------------------------------------------------------ set-up
    def before_train(self):
        exp = self.exp
        PM.initialize()
        PM.set_mesh(exp.model_cfg.parallel_cfg)
        set_mpu_random_seed(exp.seed)
        prof = getattr(exp, "profiler_cfg", None)
        init_timers(getattr(prof, "timing_log_level", 0), getattr(prof, "timing_use_event", True),
                    getattr(prof, "nvtx_ranges", False))
        GlobalMetrics.clear()
        if getattr(exp, "metric_cfg", None) is not None:
            exp.metric_cfg.register()
        if PM.world_rank == PM.world_size - 1 and getattr(exp.trainer_cfg, "writer_backend", None):
            try:
                self.writer = exp.build_log_writer()
            except Exception as e:
                logger.warning(f"no log writer: {e}", at=None)
        self.build_hooks(exp.trainer_cfg)
        self.call_hooks("after_init")
        self.call_hooks("before_train")
        self.setup_model()
        self.grad_manager = exp.optimizer_cfg.build_gradient_manager(self.models)
        self.build_dataloader()
        self.scheduler = exp.scheduler_cfg.build_scheduler(self.grad_manager.optimizer)
        ck = getattr(exp, "checkpoint_cfg", None)
        if ck is not None:
            self.checkpointer = ck.build_checkpointer()
            self.load_checkpoint()
        logger.info(f"trainer ready: {PM}", at=0)

    def setup_model(self):
        cfg = self.exp.model_cfg
        dev = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
        self.device = dev
        self.models = []
        for vp in range(PM.get_vpp_size()):
            PM.set_vpp_rank(vp)
            with torch.device(dev):
                m = cfg.build_model(vpp_rank=vp) if PM.get_vpp_size() > 1 else cfg.build_model()
            m.init_weights(self.exp.seed, getattr(cfg, "init_std", 0.02))
            self.models.append(Float16Module(m, cfg.params_dtype, cfg.fp32_output))
        PM.set_vpp_rank(0)

    def build_dataloader(self):
        exp = self.exp
        ends = PM.is_pipeline_first_stage(True) or PM.is_pipeline_last_stage(True)
        is_src = ends and PM.rank_in("TP") == 0 and PM.rank_in("CP") == 0
        if is_src:
            self.dataloader = exp.data_cfg.build_dataloader(PM.get_data_rank(), PM.get_data_world_size())
        self.data_iterators = [iter(self.dataloader) if self.dataloader is not None else None for _ in self.models]
        if len(self.models) > 1 and self.dataloader is not None:
            it = iter(self.dataloader)
            self.data_iterators = [it for _ in self.models]
        self.train_iters = exp.trainer_cfg.train_iters
        if self.train_iters is None:
            n = len(self.dataloader) if self.dataloader is not None and hasattr(self.dataloader, "__len__") else 0
            t = torch.tensor([n * PM.get_data_world_size() // exp.trainer_cfg.global_batch_size], dtype=torch.int64,
                             device=self.device)
            if torch.distributed.is_initialized():
                torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
            self.train_iters = int(t.item())

    # ------------------------------------------------------------------ loop
    def _start_watchdog(self):
        pc = getattr(self.exp, "profiler_cfg", None)
        every, stall = getattr(pc, "kernel_watchdog_s", None), getattr(pc, "stall_watchdog_s", None)
        if not every and not stall:
            return None
        from ..utils.watchdog import KernelWatchdog

        return KernelWatchdog(interval_s=float(every or min(stall / 4, 10.0)), stall_s=stall).start()

    def train_loop(self):
        tc = self.exp.trainer_cfg
        timers = get_timers()
        self._t_last = time.perf_counter()
        self._watchdog = self._start_watchdog()
        try:
            self._train_iterations(tc, timers)
        except KeyboardInterrupt:
            if self._watchdog is not None and self._watchdog.tripped.is_set():
                raise RuntimeError(self._watchdog.error) from None   # the watchdog interrupted the main thread
            raise
        finally:
            if self._watchdog is not None:
                self._watchdog.stop()

    def _train_iterations(self, tc, timers):
        first = self.iteration
        while self.iteration < self.train_iters:
            with timers.record("iteration", 0):
                self.train_step()                  # runs the before_step / after_step hooks itself
            if self.iteration == first and torch.cuda.is_available():
                torch.cuda.empty_cache()           # buffers that only the first step needed (workspace sizing, init)
            self.iteration += 1
            if self._watchdog is not None:
                self._watchdog.beat()
                self._watchdog.raise_if_tripped()
            if self.iteration % tc.log_interval == 0:
                self.training_log()
            ck = getattr(self.exp, "checkpoint_cfg", None)
            if ck is not None and ck.save_interval and self.iteration % ck.save_interval == 0:
                self.save_checkpoint()

    def num_microbatches(self) -> int:
        tc = self.exp.trainer_cfg
        n = tc.global_batch_size // PM.get_data_world_size() // tc.micro_batch_size
        if n < 1:
            raise ValueError("global_batch_size smaller than data-parallel size x micro_batch_size")
        return n

    def train_step(self):
        exp, tc = self.exp, self.exp.trainer_cfg
        timers = get_timers()
        gm = self.grad_manager
        gm.zero_grad()
        gm.wait_param_gather()
        n_micro = self.num_microbatches()
        sched = exp.model_cfg.get_pp_scheduler()
        sched.configure(self.models, self.data_iterators,
                        data_sync_fn=lambda it: tc.sync_get_data(it),
                        data_proc_fn=exp.data_cfg.preprocess, loss_fn=tc.loss_func, training=True)
        # optimizer state (fp32 masters and moments) waits on the host while activations need the memory
        offload = bool(getattr(tc, "offload_optimizer_state", False)) and hasattr(gm, "offload_state")
        with timers.record("forward-backward", 1):
            # the step hooks run inside the step, as in the reference (core/trainers/lm_trainer.py:203-204, 257-259),
            # so that code which drives train_step() itself gets them too
            self.call_hooks("before_step")
            if offload:
                CMT.mark("before_cpu_offload_optimizer_state")
                with timers.record("optimizer-offload", 2):
                    gm.offload_state()
                CMT.mark("after_cpu_offload_optimizer_state")
            sched.run(n_micro)
        CMT.mark("after_forward_backward")
        if getattr(tc, "empty_unused_memory_level", 0) >= 1 and torch.cuda.is_available():
            torch.cuda.empty_cache()
        if offload:
            with timers.record("optimizer-backload", 2):
                gm.reload_state()
            CMT.mark("after_cpu_backload_optimizer_state")
        with timers.record("optimizer-step", 1):
            ok, grad_norm, zeros = gm.step()
        CMT.mark("after_optimizer_step")
        GlobalMetrics.grad_norm.add(grad_norm)
        if zeros is not None:
            GlobalMetrics.grad_zeros.add(zeros)
        for m in self.models:
            um = unwrap_model(m)
            if hasattr(um, "after_optimizer_step"):
                um.after_optimizer_step()
        tokens = tc.global_batch_size * tc.global_seq_length
        self.consumed_samples += tc.global_batch_size
        self.scheduler.step(exp.scheduler_cfg.increment(tc.global_batch_size, tokens)
                            if hasattr(exp.scheduler_cfg, "increment") else 1)
        if getattr(tc, "empty_unused_memory_level", 0) >= 2 and torch.cuda.is_available():
            torch.cuda.empty_cache()               # level 2: also after the update
        with timers.record("after-step-hooks", 1):
            self.call_hooks("after_step")
        CMT.mark("after_step_hooks")
        return ok

    def training_log(self):
        tc = self.exp.trainer_cfg
        now = time.perf_counter()
        if torch.cuda.is_available():
            torch.cuda.synchronize()
            native.raise_if_kernel_error()
            raise_if_nonfinite()
            now = time.perf_counter()
        dt = (now - self._t_last) / tc.log_interval
        self._t_last = now
        GlobalMetrics.iteration_time.add(dt)
        metrics = GlobalMetrics.reduce_all()
        skipped = self.grad_manager.skipped_steps() if hasattr(self.grad_manager, "skipped_steps") else 0
        metrics["N-skipped"] = skipped
        # run-level counters next to the per-interval metrics, as the reference writes them (core/trainers/
        # lm_trainer.py:292-298)
        metrics["batch-size"] = tc.global_batch_size
        metrics["world-size"] = PM.world_size
        metrics["N-samples"] = self.consumed_samples
        metrics["N-tokens"] = self.consumed_samples * tc.global_seq_length
        tokens = tc.global_batch_size * tc.global_seq_length
        tps_card = tokens / dt / max(PM.world_size, 1)
        logs = tc.make_logs(self.iteration, metrics, self.writer)
        line = (f"iter {self.iteration}/{self.train_iters} | consumed samples {self.consumed_samples} | "
                f"{dt * 1e3:.1f} ms/iter | tokens-per-second-per-card {tps_card:.1f} | "
                f"lr {self.scheduler.cur_lr:.3E} | global batch size {tc.global_batch_size} | #skipped-iters {skipped} | "
                f"grad-norm {float(metrics.get('grad_norm', 0.0)):.3f} | lm_loss {logs.get('lm_loss', 'n/a')}")
        self.last_metrics = metrics                        # everything that was reduced for this log line
        self.history.append({"iteration": self.iteration, "ms_per_iter": dt * 1e3,
                             "lm_loss": float(metrics["lm_loss"]) if "lm_loss" in metrics else None,
                             "grad_norm": float(metrics.get("grad_norm", 0.0))})
        logger.info(line, at=-1)
        tl = get_timers()
        if tl.log_level > 0:
            logger.info(tl.log_string(normalizer=tc.log_interval), at=0)

    # ------------------------------------------------------------------ checkpoints
    def set_autoresume(self) -> bool:
        """When ``auto_resume`` is on and this job has written a complete checkpoint before, point the configuration
        at it: ``load_path`` = the latest checkpoint, every load option on (a run configured to start from someone
        else's weights without their optimizer must still resume its OWN optimizer, scheduler and data position),
        no safetensors.  Returns whether it did.  Reference: core/trainers/lm_trainer.py:415-436."""
        ck = self.exp.checkpoint_cfg
        latest = self.checkpointer.latest() if ck.auto_resume and self.checkpointer is not None else None
        if latest is None:
            return False
        logger.info(f"AutoResume from: {latest}", at=0)
        if ck.load_path and ck.load_path != latest:
            logger.warning(f'AutoResume is overwriting checkpoint_cfg.load_path! Was: "{ck.load_path}"', at=0)
        ck.load_path = latest
        ck.load_option.all()
        ck.load_safetensors = None
        return True

    def load_checkpoint(self):
        ck = self.exp.checkpoint_cfg
        path = ck.load_path if self.set_autoresume() else None
        hf_dir = ck.load_safetensors
        if hf_dir is True:  # the HF view that a native checkpoint carries beside it
            hf_dir = os.path.join(ck.load_path, "hf")
        if path is None and ck.load_path and not ck.load_safetensors:
            path = ck.load_path
        if path is None:
            if hf_dir:
                from ..checkpointing.hf_checkpoint import load_safetensors_into

                for m in self.models:
                    load_safetensors_into(unwrap_model(m), hf_dir, strict=bool(getattr(ck, "strict_load_model", True)))
                if hasattr(self.grad_manager, "refresh_masters_from_params"):
                    self.grad_manager.refresh_masters_from_params()   # the fp32 masters follow the loaded weights
            return
        state = self.checkpointer.load_ckpt(path, self.models, self.grad_manager, self.scheduler, self.dataloader)
        if state and ck.load_option.iter:
            self.iteration = int(state.get("iteration", 0))
            self.history = state.get("history", [])
            self.consumed_samples = int(state.get("consumed_samples", 0))

    def save_checkpoint(self, sync: bool = False):
        if self.checkpointer is None:
            return
        extra = {"exp": self.exp.to_dict(rep=True), "history": self.history, "iteration": self.iteration,
                 "consumed_samples": self.consumed_samples}
        self.checkpointer.save_ckpt(self.iteration, self.models, self.grad_manager, self.scheduler, self.dataloader,
                                    extra, sync=sync)

    def after_train(self):
        self.call_hooks("after_train")
        ck = getattr(self.exp, "checkpoint_cfg", None)
        if self.checkpointer is not None and ck is not None and ck.save_interval:
            self.save_checkpoint(sync=True)
            self.checkpointer.join()
        if self.writer is not None:
            self.writer.close()
