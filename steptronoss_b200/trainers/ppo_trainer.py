"""PPO-style RL trainer: rollouts from the flow controller, reference / actor / critic passes over packed
samples, critic and actor updates, with every role swapped in and out of device memory around its phase.

Reference: ``steptronoss/core/trainers/ppo_trainer.py:51-844``.  One iteration:

1. ``flow_controller.get_train_samples()`` (rank 0) -> broadcast -> reward / generation metrics -> filter;
2. group into packed sequences of at most ``global_seq_length`` tokens, balanced over the data ranks;
3. forward-only passes fill ``ref_logprobs`` (reference policy), ``actor_logprobs`` (current policy) and the
   values -> GAE advantages / returns (or group-relative advantages when there is no critic);
4. critic epochs, advantage normalisation over the DP group, actor epochs (skipped while the critic warms up);
5. dump the requested sample fields, log, checkpoint every role plus the flow state.
"""
from __future__ import annotations

import os
import random
import time

import torch

from ..data.nextable import Nextable
from ..exp.rl import PackedPPOSamples, PPOSample
from ..parallel.state import PM, set_mpu_random_seed
from ..utils.dist_utils import broadcast_tensors
from ..utils.general import balanced_list_split, list_split, recur_to, sync_point
from ..utils.logger import logger
from ..utils.memory_tracker import CMT
from ..utils.metrics import GlobalMetrics
from ..utils.rl_utils import RaggedPPOSampleDumper
from ..utils.timers import init_timers
from .base_trainer import BaseTrainer
from .packed_model import PackedModel


def _raise_if_kernel_error() -> None:
    """Surface a kernel's bounded-wait failure (unreduced shard, overfull expert buffer) before its consequences
    are logged or written to a checkpoint."""
    if torch.cuda.is_available():
        from ..ops import native

        torch.cuda.synchronize()
        native.raise_if_kernel_error()


class TrainerPromptStream(Nextable):
    """The prompt loader seen through the experiment's ``preprocess`` (what the flow controller pulls from)."""

    def __init__(self, dataloader, proc=None):
        self.dataloader, self.proc = dataloader, proc
        self._it = None

    def __next__(self):
        if self._it is None:
            self._it = iter(self.dataloader)
        item = next(self._it)
        return self.proc(item) if self.proc is not None else item

    def state_dict(self):
        return self.dataloader.state_dict() if hasattr(self.dataloader, "state_dict") else None

    def load_state_dict(self, sd):
        if sd is not None and hasattr(self.dataloader, "load_state_dict"):
            self.dataloader.load_state_dict(sd)


def get_normalizer(x: torch.Tensor):
    """Mean and std of ``x`` over the DP group; a NaN/Inf in any rank's values is an error (a silent NaN here would
    poison every advantage of the batch)."""
    stats = torch.stack([x.sum(), (x * x).sum(), torch.as_tensor(float(x.numel()), device=x.device)]).double()
    group = PM.group_of("DP")
    if group is not None:
        torch.distributed.all_reduce(stats, group=group)
    mean = stats[0] / stats[2]
    var = (stats[1] / stats[2] - mean * mean).clamp_min(0)
    if not bool(torch.isfinite(stats[:2]).all()):
        raise ValueError(f"get_normalizer: non-finite result (mean={float(mean)}, std={float(var.sqrt())}); "
                         f"the input holds NaN or Inf")
    return mean.float(), var.sqrt().float()


class PPOTrainer(BaseTrainer):
    def __init__(self, exp):
        super().__init__(exp)
        self.ppo_cfg = exp.trainer_cfg
        self.checkpointer = None
        self.flow_controller = None
        self.actor = self.critic = self.reference_model = None
        self.start_iteration = self.actor_iteration = self.critic_iteration = 0
        self.writer = None
        self.history: list = []

    # ------------------------------------------------------------------------------------ set-up
    def initialize_dist(self):
        exp = self.exp
        PM.initialize()
        PM.set_mesh(exp.actor_model_cfg.parallel_cfg)
        set_mpu_random_seed(exp.seed)
        prof = getattr(exp, "profiler_cfg", None)
        self.timers = init_timers(getattr(prof, "timing_log_level", 0), getattr(prof, "timing_use_event", True),
                    getattr(prof, "nvtx_ranges", False))
        GlobalMetrics.clear()
        exp.metric_cfg.register()
        if PM.world_rank == PM.world_size - 1 and getattr(exp.trainer_cfg, "writer_backend", None):
            try:
                self.writer = exp.build_log_writer()
            except Exception as e:
                logger.warning(f"no log writer: {e}", at=None)
        self.build_hooks(exp.trainer_cfg)
        self.call_hooks("after_init")
        self.call_hooks("before_train")

    def before_train(self):
        self.initialize_dist()
        self.build_models_and_flow_controller()

    def after_train(self):
        ck = self.exp.checkpoint_cfg
        if ck.save_interval and self.iteration != 0 and self.checkpointer is not None:
            self.save_checkpoint(sync=True)
        self.call_hooks("after_train")

    def _build_role(self, name: str, model_cfg, gm_cfg, sched_cfg, training: bool) -> PackedModel:
        role_ck = getattr(self.exp.checkpoint_cfg, name if name != "reference_model" else "reference")
        pm = PackedModel(self.ppo_cfg, model_cfg, gm_cfg, sched_cfg, training=training, name=name, seed=self.exp.seed)
        path = role_ck.load_path
        if path:
            old = self.exp.checkpoint_cfg.load_option
            self.exp.checkpoint_cfg.load_option = role_ck.load_option
            try:
                extra = self.checkpointer.load_ckpt(path, pm.models, pm.grad_manager, pm.scheduler, None)
            finally:
                self.exp.checkpoint_cfg.load_option = old
            pm.loaded_iteration = int(extra.get("iteration", 0)) if extra else 0
        elif role_ck.load_safetensors:
            from ..checkpointing.hf_checkpoint import load_safetensors_into
            from ..models.module import unwrap_model

            for m in pm.models:
                load_safetensors_into(unwrap_model(m), role_ck.load_safetensors,
                                      strict=role_ck.strict_load_model is not False)
            if pm.grad_manager is not None:
                pm.grad_manager.refresh_masters_from_params()
        return pm

    def set_autoresume(self) -> bool:
        """When ``auto_resume`` is on and this job has written a complete checkpoint before: every role's
        ``load_path`` becomes its directory in that checkpoint, every load option is switched on and safetensors
        sources are dropped, so that a job set up to start from foreign weights resumes its own optimizers,
        schedulers and flow state.  Reference: core/trainers/ppo_trainer.py:752-784."""
        ck = self.exp.checkpoint_cfg
        latest = self._resume_dir()
        if latest is None:
            return False
        logger.info(f"AutoResume from: {latest}", at=0)
        if ck.load_path and ck.load_path != latest:
            logger.warning(f'AutoResume is overwriting checkpoint_cfg.load_path! Was: "{ck.load_path}"', at=0)
        ck.load_path, ck.load_safetensors = latest, None
        ck.load_option.all()
        for role in ("actor", "critic", "reference"):
            rc = getattr(ck, role, None)
            if rc is not None and os.path.isdir(os.path.join(latest, role)):   # a role the checkpoint does not hold
                rc.load_path, rc.load_safetensors = os.path.join(latest, role), None   # keeps its original source
                rc.load_option.all()
        return True

    def _resume_dir(self, sub: str | None = None) -> str | None:
        ck = self.exp.checkpoint_cfg
        if not ck.auto_resume or self.checkpointer is None:
            return None
        latest = self.checkpointer.latest()
        if latest is None:
            return None
        return os.path.join(latest, sub) if sub else latest

    def build_flow_controller(self):
        """Hook for tests and custom generation back ends."""
        return self.ppo_cfg.flow_cfg.build_flow_controller()

    def build_models_and_flow_controller(self):
        exp = self.exp
        self.checkpointer = exp.checkpoint_cfg.build_checkpointer()
        self.set_autoresume()
        with self.timers.record("build_actor_model", 1):
            self.actor = self._build_role("actor", exp.actor_model_cfg, exp.actor_grad_manager_cfg,
                                          exp.actor_scheduler_cfg, True)
            self.actor_iteration = getattr(self.actor, "loaded_iteration", 0)
            self.actor.offload_model()
            self.actor.offload_state()
        CMT.mark("after_build_actor")
        if exp.critic_model_cfg is not None and self.ppo_cfg.use_critic:
            with self.timers.record("build_critic_model", 1):
                self.critic = self._build_role("critic", exp.critic_model_cfg, exp.critic_grad_manager_cfg,
                                               exp.critic_scheduler_cfg, True)
                self.critic_iteration = getattr(self.critic, "loaded_iteration", 0)
                self.critic.offload_model()
                self.critic.offload_state()
        elif self.ppo_cfg.use_critic:
            raise ValueError("Critic model must be provided for PPO training (or set trainer_cfg.use_critic=False)")
        CMT.mark("after_build_critic")
        if not self.ppo_cfg.skip_forward_reference:
            with self.timers.record("build_reference_model", 1):
                self.reference_model = self._build_role("reference_model", exp.actor_model_cfg, None, None, False)
                self.reference_model.offload_model()
        CMT.mark("after_build_reference")
        if PM.world_rank == 0:
            os.makedirs(exp.checkpoint_cfg.save_path, exist_ok=True)
        flow_state, top = None, self._resume_dir()
        if top is not None:
            import pickle

            data_file = os.path.join(top, "data.pkl")
            if PM.world_rank == 0 and os.path.exists(data_file):
                with open(data_file, "rb") as f:
                    flow_state = pickle.load(f)
            it_file = os.path.join(top, "trainer_iteration")
            if os.path.exists(it_file):
                self.start_iteration = int(open(it_file).read()) + 1
        stream = None
        if PM.world_rank == 0:
            stream = TrainerPromptStream(exp.data_cfg.build_dataloader(), getattr(exp.data_cfg, "preprocess_prompt", None))
        self.flow_controller = self.build_flow_controller()
        self.flow_controller.start(dataloader=stream, model=self.actor.models, state_dict=flow_state)

    # ------------------------------------------------------------------------------------ loop
    def train_loop(self):
        tc, ck = self.ppo_cfg, self.exp.checkpoint_cfg
        self.iteration = self.start_iteration
        sync_point("before the start of training step")
        while self.iteration < tc.train_iters:
            t0 = time.perf_counter()
            self.call_hooks("before_step")
            if self.eval_due():
                self.eval()
            self.train_step()
            self.call_hooks("after_step")
            if torch.cuda.is_available():
                torch.cuda.synchronize()
            GlobalMetrics.iteration_time.add(time.perf_counter() - t0)
            self.training_log()
            if ck.save_interval and self.iteration % ck.save_interval == 0 and self.iteration > self.start_iteration:
                self.save_checkpoint()
            self.iteration += 1

    # ------------------------------------------------------------------------------------ rollouts
    def adapt_trajs_to_samples(self, rollouts: list) -> list:
        out = []
        for s in rollouts:
            s.trajectory = torch.as_tensor(s.trajectory, dtype=torch.long)
            s.is_gen_mask = torch.as_tensor(s.is_gen_mask, dtype=torch.bool)
            if s.logprobs is not None:
                s.logprobs = torch.as_tensor(s.logprobs, dtype=torch.float32)
            else:
                s.logprobs = torch.zeros(int(s.is_gen_mask.sum()), dtype=torch.float32)
            if s.meta is None:
                s.meta = {}
            sample = PPOSample(**dict(s.items()))
            gt = s.meta.get("ground_truth")                 # what the prompt's data row says about scoring and origin
            if isinstance(gt, dict):
                sample.ground_truth = gt
            out.append(sample)
        return out

    def generate_trajectory(self) -> list:
        """The rollouts of this iteration, identical on every rank."""
        with self.timers.record("generate_trajectory", 1):
            samples = self.flow_controller.get_train_samples()
            if PM.world_rank == 0:
                samples = self.adapt_trajs_to_samples(samples)
            if PM.world_size > 1:
                samples = broadcast_tensors(samples, src=0, group=None)
        return samples

    @staticmethod
    def _group_samples(samples: list, max_seq_len: int = 8192, divisable_by: int = 1):
        """Greedy packing in arrival order; over-long samples are dropped, trailing groups are dropped so that
        the group count is a multiple of ``divisable_by``."""
        groups, sizes = [[]], [0]
        for s in samples:
            n = len(s.trajectory)
            if n > max_seq_len:
                continue
            if sizes[-1] + n <= max_seq_len:
                groups[-1].append(s)
                sizes[-1] += n
            else:
                groups.append([s])
                sizes.append(n)
        if not groups[0]:
            groups, sizes = [], []
        extra = len(groups) % divisable_by
        if extra:
            groups, sizes = groups[:-extra], sizes[:-extra]
        return groups, sizes

    def data_balance_and_pack(self, all_samples: list) -> list:
        GlobalMetrics.unpacked_samples.add(float(len(all_samples)))
        dw = PM.get_data_world_size()
        d = dw * (PM.size_of("PP") if PM.get_vpp_size() > 1 else 1)
        groups, sizes = self._group_samples(all_samples, self.ppo_cfg.global_seq_length, d)
        logger.info(f"Global Rollout: pack({len(all_samples)}) -> {len(groups)}", at=-1)
        GlobalMetrics.packed_samples.add(float(len(groups)))
        if len(groups) < dw:
            raise RuntimeError("Not enough rollouts to give every data rank a packed sequence")
        mine = balanced_list_split(groups, sizes, dw)[PM.get_data_rank()]
        packed = [PackedPPOSamples.from_samples(g) for g in mine]
        random.Random(1234).shuffle(packed)
        return packed

    # ------------------------------------------------------------------------------------ forward-only passes
    def _forward_only(self, role: PackedModel, samples: list, fn):
        def loss_fn(data, outputs, loss_scale=1.0):
            fn(data["_samples"], outputs)
            return None

        with torch.no_grad():
            role.forward_backward(samples, self.ppo_cfg.preprocess_generated, loss_fn=loss_fn, training=False)
        return samples

    def get_reference(self, samples: list) -> list:
        def fill(packed, logits):
            mask = packed.is_gen_mask.reshape(-1).to(logits.device).bool()
            packed.ref_logprobs = self.ppo_cfg.token_logprobs(packed, logits)[mask].contiguous()

        with self.timers.record("get_reference", 1):
            return self._forward_only(self.reference_model, samples, fill)

    def get_actor_logprob(self, samples: list) -> list:
        def fill(packed, logits):
            mask = packed.is_gen_mask.reshape(-1).to(logits.device).bool()
            lp = self.ppo_cfg.token_logprobs(packed, logits, self.ppo_cfg.policy_actor_temperature)
            packed.actor_logprobs = lp[mask].contiguous()

        with self.timers.record("get_actor_logprob", 1):
            self._forward_only(self.actor, samples, fill)
        self.ppo_cfg.log_sampling_logprob_metrics(samples)
        return samples

    def get_values_advantages(self, samples: list) -> list:
        def fill(packed, values):
            v = values.reshape(values.shape[0], -1)[:, 0]
            if PM.size_of("CP") > 1:
                from ..parallel.context_parallel import gather_from_balanced_cp_region

                v = gather_from_balanced_cp_region(v)  # GAE needs the whole sequence in order
            self.ppo_cfg.get_advantage_and_returns(ragged_samples=packed, ragged_values=v)

        with self.timers.record("get_values_advantages", 1):
            return self._forward_only(self.critic, samples, fill)

    def normalize_advantages(self, samples: list) -> list:
        if not PM.is_pipeline_last_stage(ignore_virtual=True) or not samples:
            return samples
        dev = "cuda" if torch.cuda.is_available() else "cpu"
        for s in samples:
            s.advantages = s.advantages.to(dev)
        adv = torch.cat([s.advantages for s in samples])
        GlobalMetrics.advantage_max.add(adv.max())
        GlobalMetrics.advantage_min.add(adv.min())
        mean, std = get_normalizer(adv)
        GlobalMetrics.advantage_std.add(std.clone())
        std = std.clamp_min(0.01)
        for s in samples:
            s.advantages = (s.advantages - mean) / std
            GlobalMetrics.advantage_mean.add(s.advantages.mean())
            GlobalMetrics.advantage_abs_mean.add(s.advantages.abs().mean())
        return samples

    def make_div_pp(self, data: list) -> list:
        if PM.get_vpp_size() > 1:
            pp = PM.size_of("PP")
            assert len(data) >= pp, "No Enough Data!"
            data = data[: len(data) // pp * pp]
        return data

    def chunk_my_samples(self, my_samples: list, fix_iters: int | None = None) -> list:
        assert fix_iters
        min_chunk = PM.size_of("PP") if PM.get_vpp_size() > 1 else 1
        return list_split(my_samples, split=max(1, min(fix_iters, len(my_samples) // min_chunk)))

    # ------------------------------------------------------------------------------------ one iteration
    def train_step(self):
        cfg = self.ppo_cfg
        CMT.mark("start_of_iter")
        self.actor.offload_model()
        self.actor.offload_state()
        all_samples = self.generate_trajectory()
        cfg.log_generation_metrics(all_samples)
        cfg.log_reward_metrics(all_samples)
        all_samples = cfg.filter_samples(all_samples)
        my_samples = self.data_balance_and_pack(all_samples)
        logger.info(f"Get {len(my_samples)} packed-samples for each DP.", at=-1)
        if not cfg.skip_forward_reference:
            self.reference_model.backload_model()
            my_samples = self.get_reference(my_samples)
            self.reference_model.offload_model()
        if not cfg.skip_forward_actor:
            self.actor.backload_model()
            my_samples = self.get_actor_logprob(my_samples)
            self.actor.offload_model()
        if self.critic is not None:
            self.critic.backload_model()
            if not cfg.onvalue_gae:
                my_samples = self.get_values_advantages(my_samples)
        else:
            for s in my_samples:
                cfg.group_relative_advantages(s)
        if cfg.offload_data:
            my_samples = recur_to(my_samples, "cpu")
        if self.critic is not None:
            self.critic.backload_state()
            critic_chunks = self.chunk_my_samples(my_samples, cfg.fix_iters_critic)
            with self.timers.record("critic_train", 1):
                for ep in range(cfg.critic_epoch):
                    GlobalMetrics.inner_iteration.add(float(len(critic_chunks)))
                    logger.info(f"CriticTrain: Ep={ep} iters={len(critic_chunks)}", at=-1)
                    for chunk in critic_chunks:
                        if cfg.onvalue_gae:
                            self.get_values_advantages(chunk)
                        self.critic.forward_backward(self.make_div_pp(chunk), cfg.preprocess_generated,
                                                     loss_fn=cfg.critic_loss_func, training=True,
                                                     offload_opt_while_forward=bool(cfg.offload_optimizer_state),
                                                     offload_data=cfg.offload_data)
                        _, grad_norm, zeros = self.critic.optimizer_step()
                        GlobalMetrics.critic_grad_norm.add(grad_norm)
                        self.critic_iteration += 1
            if cfg.onvalue_gae:
                my_samples = [s for chunk in critic_chunks for s in self.make_div_pp(chunk)]
        with self.timers.record("normalize_advantages", 1):
            my_samples = self.normalize_advantages(my_samples)
        if self.critic is not None:
            self.critic.offload_model()
            self.critic.offload_state()
        self.actor.backload_model()
        self.actor.backload_state()
        actor_chunks = self.chunk_my_samples(my_samples, cfg.fix_iters)
        with self.timers.record("actor_train", 1):
            for ep in range(cfg.actor_epoch):
                logger.info(f"ActorTrain: Ep={ep} iters={len(actor_chunks)}", at=-1)
                for chunk in actor_chunks:
                    learn = self.critic is None or self.actor_iteration >= cfg.critic_warmup_iters
                    self.actor.forward_backward(self.make_div_pp(chunk), cfg.preprocess_generated,
                                                loss_fn=cfg.actor_loss_func, training=learn,
                                                offload_opt_while_forward=bool(cfg.offload_optimizer_state),
                                                offload_data=cfg.offload_data)
                    if learn:
                        _, grad_norm, zeros = self.actor.optimizer_step()
                        GlobalMetrics.actor_grad_norm.add(grad_norm)
                    self.actor_iteration += 1
        self.actor.offload_model()
        self.actor.offload_state()
        if cfg.dump_sample_keys and cfg.record_rollout:
            with self.timers.record("dump_all_samples", 1):
                self.dump_all_samples(my_samples)

    def dump_all_samples(self, my_samples: list) -> None:
        data = RaggedPPOSampleDumper()(recur_to(my_samples, "cpu"), self.ppo_cfg.dump_sample_keys)
        path = os.path.join(self.exp.checkpoint_cfg.save_path, f"ppo_samples_it{self.iteration}")
        os.makedirs(path, exist_ok=True)
        PM.barrier()
        if PM.is_pipeline_last_stage(ignore_virtual=True) and PM.rank_in("TP") == 0 and PM.rank_in("CP") == 0:
            torch.save(data, os.path.join(path, f"{PM.world_rank}.pt"))

    def step_log(self, prefix: str, step: int, **kw):
        if self.writer:
            for k, v in kw.items():
                self.writer.add_scalar(f"{prefix}/{k}", float(v), global_step=step)
        logger.info(f"{prefix}@it{step}: " + " | ".join(f"{k}: {float(v):.3e}" for k, v in kw.items()), at=-1)

    def training_log(self):
        tc = self.ppo_cfg
        _raise_if_kernel_error()
        metrics = GlobalMetrics.reduce_all()
        logs = {"iter": f"{self.iteration:8d}/{tc.train_iters:8d}"}
        for k in ("reward_mean", "ppo_loss", "critic_loss", "actor_grad_norm", "rollout_avg_tokens"):
            if k in metrics:
                logs[k] = f"{float(metrics[k]):.4f}"
        user = tc.make_logs(self.iteration, metrics, self.writer)
        if user:
            logs.update(user)
        self.history.append({"iteration": self.iteration, **{k: float(v) for k, v in metrics.items()
                                                             if torch.is_tensor(v) and v.numel() == 1
                                                             or isinstance(v, (int, float))}})
        logger.info(" | ".join(f"{k}: {v}" for k, v in logs.items()), at=-1)
        CMT.report_over_world() if hasattr(CMT, "report_over_world") else None

    def eval_due(self) -> bool:
        """Evaluation runs before the training step of every ``eval_interval``-th iteration (the very first one
        unless ``skip_first_eval``), when the experiment has an ``eval_cfg``."""
        tc = self.ppo_cfg
        every = getattr(tc, "eval_interval", None)
        if not every or getattr(self.exp, "eval_cfg", None) is None:
            return False
        if self.iteration % every:
            return False
        return not (self.iteration == 0 and getattr(tc, "skip_first_eval", False))

    def eval(self):
        """Run the experiment's benchmarks against the inference servers (they hold the current policy after the
        last weight push) on the logging rank; the scores go to the log and the writer.  Other ranks wait."""
        cfg = getattr(self.exp, "eval_cfg", None)
        summary = None
        if cfg is not None and PM.world_rank == PM.world_size - 1:
            summary = cfg.eval()
            for bench, res in (summary or {}).items():
                metric = res.get("metric", {}) if isinstance(res, dict) else {}
                for k, v in metric.items():
                    if isinstance(v, (int, float)):
                        logger.info(f"eval @ iteration {self.iteration}: {bench}/{k} = {v:.4f}", at=None)
                        if self.writer is not None:
                            self.writer.add_scalar(f"eval/{bench}/{k}", v, self.iteration)
        sync_point("evaluation done")
        return summary

    # ------------------------------------------------------------------------------------ checkpoints
    def save_checkpoint(self, sync: bool = False):
        ck = self.checkpointer
        ck.join()
        _raise_if_kernel_error()
        sync_point("ready for dump")
        roles = [("actor", self.actor, self.actor_iteration), ("critic", self.critic, self.critic_iteration),
                 ("reference", self.reference_model, self.iteration)]
        for name, role, it in roles:
            if role is None:
                continue
            role.backload_model()
            role.backload_state()
            ck.save_ckpt(self.iteration, role.models, role.grad_manager, role.scheduler, None,
                         {"iteration": it, "role": name}, sync=True, sub_name=name, mark_latest=False)
            role.offload_model()
            role.offload_state()
        if self.flow_controller is not None:
            self.flow_controller.weight_dumped()
        top = ck.iteration_dir(self.iteration)
        if PM.world_rank == 0:
            with open(os.path.join(top, "trainer_iteration"), "w") as f:
                f.write(str(self.iteration))
        ck.save_ckpt(self.iteration, [], None, None, self.flow_controller,
                     {"exp": self.exp.to_dict(rep=True), "iteration": self.iteration}, sync=True)
