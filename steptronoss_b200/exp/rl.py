"""PPO-style reinforcement learning: sample containers, role checkpoints, metrics, flow-controller and
trainer configuration.

Reference: ``steptronoss/exp/rl.py:36-944``.  Trajectories come back from the generation side-car as
:class:`EnvTrajectory`; the trainer turns them into :class:`PPOSample`, packs them into
:class:`PackedPPOSamples` (one packed sequence per micro-batch, the batch contract of the decoder) and runs
the reference / actor / critic passes over them.  The reference leaves advantage estimation and the two
losses to the experiment file; here the trainer config carries working defaults (GAE over the response
tokens, clipped PPO surrogate with optional KL terms, clipped value loss) that an experiment may override.
"""
from __future__ import annotations

import os

import torch

from ..config import Config, DataClass, Ref
from .base_exp import BaseExp, DataConfig, GradientManagerConfig, Megatron3DParallelModelConfig, MetricConfig, \
    ProfilerConfig, TrainerConfig
from .checkpointing import CheckpointConfig, LoadOptions
from .inference import VLLMDeployConfig
from .lr_schedulers import SchedulerConfig


class StopType:
    MAX_LEN = 1
    MAX_DECODE = 2
    STOP_TOKEN = 3
    STOP_STRING = 4
    STOP_PARTIAL = 5


class EnvTrajectory(DataClass):
    """One rollout with its reward.  ``trajectory`` = prompt + generated tokens ``(St,)``; ``logprobs`` are
    the sampling log-probabilities of the generated tokens ``(Sr,)``; ``is_gen_mask`` marks them ``(St,)``."""

    trajectory: torch.Tensor | list = None
    logprobs: torch.Tensor | list | None = None
    is_gen_mask: torch.Tensor | list = None
    meta: dict = None
    stop_type: int = StopType.STOP_TOKEN
    raw_reward: float = None

    @property
    def can_be_trained(self) -> bool:
        ok = self.raw_reward is not None and self.trajectory is not None and self.is_gen_mask is not None
        if ok and self.logprobs is not None:
            ok = int(sum(self.is_gen_mask)) == len(self.logprobs)
        return ok


class PPOSample(EnvTrajectory):
    ground_truth = {}
    prompt_id: str = None
    ref_logprobs: torch.Tensor = None
    actor_logprobs: torch.Tensor = None
    advantages: torch.Tensor = None
    returns: torch.Tensor = None
    values: torch.Tensor = None
    input_ids: torch.Tensor = None
    labels: torch.Tensor = None


class PackedPPOSamples(DataClass):
    """Several samples packed into one sequence.  Token-indexed fields are ``[1, S]`` (``S`` padded to a
    multiple of ``2*TP*CP``); response-indexed fields (``logprobs``, ``advantages`` ...) are the
    concatenation over samples of the generated positions, in ``is_gen_mask`` order (the mask is shifted
    left by one like the labels: position ``t`` predicts token ``t+1``)."""

    input_ids: torch.Tensor = None
    labels: torch.Tensor = None
    cu_seqlens: torch.Tensor = None
    cu_valid_sizes: torch.Tensor = None
    max_seq_len: torch.Tensor = None
    trajectory: torch.Tensor = None
    is_gen_mask: torch.Tensor = None
    loss_mask: torch.Tensor = None
    advantages: torch.Tensor = None
    returns: torch.Tensor = None
    values: torch.Tensor = None
    logprobs: torch.Tensor = None
    ref_logprobs: torch.Tensor = None
    actor_logprobs: torch.Tensor = None
    samples: list = None

    @classmethod
    def from_samples(cls, samples: list) -> "PackedPPOSamples":
        from ..parallel.state import PM
        from ..utils.general import pad_tensor, shift_left

        out = cls()
        labels = [shift_left(s.trajectory) for s in samples]
        masks = [shift_left(s.is_gen_mask) for s in samples]
        lens = torch.tensor([len(s.trajectory) for s in samples], dtype=torch.int32)
        cu = torch.cat([torch.zeros(1, dtype=torch.int32), torch.cumsum(lens, 0).to(torch.int32)])
        align = PM.size_of("TP") * PM.size_of("CP") * 2
        num_pad = (-int(cu[-1])) % align
        out.cu_valid_sizes = cu.clone()
        cu[-1] += num_pad
        out.cu_seqlens = cu
        out.max_seq_len = cu.diff().max()

        def pad(x, dim=0):
            return pad_tensor(x, dim=dim, to=x.shape[dim] + num_pad, value=0)

        samples[-1].is_gen_mask = pad(samples[-1].is_gen_mask)
        samples[-1].trajectory = pad(samples[-1].trajectory)
        out.trajectory = pad(torch.cat([s.trajectory[: int(n)] for s, n in zip(samples, lens)])[None], dim=1)
        out.input_ids = out.trajectory
        out.labels = pad(torch.cat(labels)[None], dim=1)
        out.is_gen_mask = pad(torch.cat(masks)[None], dim=1)
        out.logprobs = torch.cat([s.logprobs for s in samples])
        out.samples = samples
        return out


# ----------------------------------------------------------------------------------------------- configs
class RoleCheckpointConfig(Config):
    load_path: str | None = None
    load_safetensors: bool | str | None = None
    strict_load_model: bool | None = None
    load_option: LoadOptions = LoadOptions


class PPOCheckpointCfg(CheckpointConfig):
    """One load source per role; the job's own checkpoints hold all roles."""

    actor: RoleCheckpointConfig = RoleCheckpointConfig
    critic: RoleCheckpointConfig = RoleCheckpointConfig
    reference: RoleCheckpointConfig = RoleCheckpointConfig


class PPOMetricConfig(MetricConfig):
    def __init__(self):
        super().__init__()
        from ..utils.metrics import AvgMetric, GroupMetric, HistogramMetric, Metric, PercentageMetric, TextMetric

        self.reward_mean = Metric().mean("time").mean("dp")
        self.reward_max = Metric().max("time").max("dp")
        self.reward_min = Metric().min("time").min("dp")
        self.correctness = PercentageMetric().sum("world")
        self.correctness_subclass = PercentageMetric().sum("world")       # the same, split by reward function
        self.reward_func_mean = GroupMetric().mean("time").mean("world")
        self.reward_func_max = GroupMetric().mean("time").max("world")
        self.reward_func_min = GroupMetric().mean("time").min("world")
        # rewards, response lengths, truncation and log-probabilities grouped by the data file a prompt came from
        # and by its reward function
        self.reward_filename_mean = GroupMetric().mean("time").mean("world")
        self.reward_filename_max = GroupMetric().mean("time").max("world")
        self.reward_filename_min = GroupMetric().mean("time").min("world")
        self.rollout_avg_tokens_grouped = GroupMetric().mean("time").mean("world")
        self.truncated_rate_grouped = GroupMetric().mean("time").mean("world")
        self.rollout_logprob_grouped = GroupMetric().mean("time").mean("world")
        self.rollout_samples = Metric().mean("time")
        self.rollout_tokens_hist = HistogramMetric().disable()
        self.rollout_avg_tokens = Metric().mean("time")
        self.rollout_avg_solution_tokens = Metric().mean("time")
        self.rollout_avg_think_tokens = Metric().mean("time")
        self.truncated_rate = Metric().mean("time")
        self.rollout_logprob = Metric().mean("time")
        self.rollout_logprob_correct = Metric().mean("time")
        self.rollout_logprob_incorrect = Metric().mean("time")
        # per-sample means pooled over all ranks: ranks score different numbers of responses
        self.repeatness_score = AvgMetric().mean("world")
        self.repeatness_rate = AvgMetric().mean("world")
        self.repeatness_rate_correct = AvgMetric().mean("world")
        self.repeatness_rate_incorrect = AvgMetric().mean("world")
        self.actor_grad_norm = Metric().mean("time")
        self.critic_grad_norm = Metric().mean("time")
        self.kl_with_ref_dist = Metric().mean("time").mean("dp")
        self.kl_with_sample_dist = Metric().mean("time").mean("dp")
        self.ppo_loss = Metric().mean("time").mean("dp")
        self.critic_loss = Metric().mean("time").mean("dp")
        self.ppo_clip_frac = Metric().mean("time").mean("dp")
        self.value_clip_frac = Metric().mean("time").mean("dp")
        self.advantage_max = Metric().max("time").max("dp")
        self.advantage_min = Metric().min("time").min("dp")
        self.advantage_std = Metric().mean("time").mean("dp")
        self.advantage_mean = Metric().mean("time").mean("dp")
        self.advantage_abs_mean = Metric().mean("time").mean("dp")
        self.unpacked_samples = Metric().mean("time")
        self.packed_samples = Metric().mean("time")
        self.inner_iteration = Metric().sum("time")
        self.sample_filter_rate = Metric().mean("time")
        self.logprob_diff_mean = Metric().mean("time").mean("dp")
        self.logprob_diff_max = Metric().max("time").max("dp")
        # off-policy diagnostics: the policy that trains against the one that sampled (an inference engine's
        # numerics when the run is on-policy).  Quantile groups carry min, max, q01, q05, q10, q90, q95, q99.
        self.sampling_logprob_diff = Metric().mean("time").mean("dp")
        self.sampling_logprob_diff_max = Metric().max("time").max("dp")
        self.sampling_logprob_diff_quantile = GroupMetric().mean("time").mean("dp")
        self.sampling_ratio_diff = GroupMetric().mean("time").mean("dp")
        self.new_logprob = GroupMetric().mean("time").mean("dp")
        self.old_logprob = GroupMetric().mean("time").mean("dp")
        self.new_prob = GroupMetric().mean("time").mean("dp")
        self.old_prob = GroupMetric().mean("time").mean("dp")
        self.ppo_clip_count = Metric().mean("time").mean("dp")                # share of clipped tokens
        self.ppo_lower_bound_clip_count = Metric().mean("time").mean("dp")
        self.ppo_upper_bound_clip_count = Metric().mean("time").mean("dp")
        self.ratio_diff = Metric().mean("time").mean("dp")                    # mean |pi / pi_old - 1|
        self.ratio_diff_quantile = GroupMetric().mean("time").mean("dp")
        self.reverse_kl_with_sample_dist = Metric().mean("time").mean("dp")
        self.ppo_value_clip_count = Metric().mean("time").mean("dp")
        self.ppo_returns = Metric().mean("time").mean("dp")
        self.ppo_values = Metric().mean("time").mean("dp")
        self.training_generation_text = TextMetric(20)
        self.eval_generation_text = TextMetric(10)


class ActorModelConfig(Megatron3DParallelModelConfig):
    """A policy that can also be served: carries the deployment config of its inference replicas."""

    vllm_cfg: VLLMDeployConfig = VLLMDeployConfig


class CriticModelConfig(Megatron3DParallelModelConfig):
    """A decoder whose output embedding maps hidden states to one value per token."""


class RewardModelConfig(Megatron3DParallelModelConfig):
    """Same shape as the critic."""


class FlowControllerConfig(Config):
    vllm_cfg = Ref("...actor_model_cfg.vllm_cfg")
    save_path = Ref("...checkpoint_cfg.save_path", None)
    async_strategy: str = "on-policy"
    """``on-policy`` | ``one-step-off`` (or ``fully-async`` with the subclass below)."""
    genable_allow_errors: bool = False
    prompt_per_iter: int = 64
    max_concurrent_genables: int | None = None
    num_generation_workers: int | None = None

    def sanity_check(self):
        super().sanity_check()
        assert self.async_strategy in ("on-policy", "one-step-off", "fully-async")
        assert self.max_concurrent_genables is None or self.max_concurrent_genables >= 1

    def build_flow_controller(self):
        from ..generators.flow_controller import SimpleFlowController

        return SimpleFlowController(flow_cfg=self)


class FullyAsyncFlowControllerConfig(FlowControllerConfig):
    max_untrained_prompts: int = 256
    max_staleness: int = 2

    def __init__(self):
        super().__init__()
        self.async_strategy = "fully-async"

    def sanity_check(self):
        super().sanity_check()
        assert self.max_untrained_prompts + 1 >= self.prompt_per_iter

    def build_flow_controller(self):
        from ..generators.flow_controller import FullyAsyncFlowController

        return FullyAsyncFlowController(flow_cfg=self)


class PPOLikeTrainerConfig(TrainerConfig):
    flow_cfg: FlowControllerConfig = FlowControllerConfig

    def get_trainer_cls(self) -> type:
        from ..trainers.ppo_trainer import PPOTrainer

        return PPOTrainer

    build_tokenizer = Ref("..tokenizer_cfg.build_tokenizer", None)
    critic_epoch: int = 1
    actor_epoch: int = 1
    eval_interval: int | None = None
    ppo_actor_lambda: float = 0.95
    ppo_critic_lambda: float = 0.99
    ppo_gae_gamma: float = 1.0
    advantage_clip_min: float = -5
    advantage_clip_max: float = 4.5
    critic_value_clip: float | None = 0.2
    """range of the clipped value loss around the values of the sampling pass; None or 0: plain MSE"""
    ppo_clip: float = 0.2
    reward_clip: float = 20
    sample_kl_loss_coeff: float = 0.0
    ref_kl_loss_coeff: float = 0.05
    ref_kl_penalty_coeff: float = 0.05
    dual_clip_eps: float = 1.5
    critic_warmup_iters: int = 100
    record_rollout: bool = False
    fix_iters: int | None = 1
    fix_iters_critic = Ref(".fix_iters")
    policy_actor_temperature: float = 1.0
    onvalue_gae: bool = False
    offload_data: bool = False
    offload_optimizer_state: bool | str = False
    skip_first_eval: bool = False
    skip_forward_reference: bool = False
    skip_forward_actor: bool = False
    use_offpolicy_without_is: bool = False
    use_critic: bool = True
    """Without a critic the advantage of a response is its reward minus the mean reward of its prompt group."""
    dump_sample_keys: list = ["trajectory", "logprobs", "is_gen_mask", "ground_truth", "raw_reward"]

    def sanity_check(self):
        super().sanity_check()
        if self.skip_forward_reference:
            assert self.ref_kl_loss_coeff == 0 and self.ref_kl_penalty_coeff == 0, \
                "Cannot skip get_ref_logprob when need KL regulation."
        if self.skip_forward_actor:
            assert (self.fix_iters == 1 and self.actor_epoch == 1) or self.use_offpolicy_without_is
        assert self.offload_optimizer_state in (True, False, "momentum")
        known = set(PPOSample()._defined_attributes)
        bad = set(self.dump_sample_keys or []) - known
        if bad:
            raise KeyError(f"Unsupported Key: {bad}!! supported keys are: {sorted(known)}")
        if "wandb" in (self.writer_backend or []):
            assert os.getenv("WANDB_API_KEY") is not None

    # ---------------------------------------------------------------------------- data movement
    def is_data_source(self) -> bool:
        from ..parallel.state import PM

        return PM.is_pipeline_first_stage(ignore_virtual=True) or PM.is_pipeline_last_stage(ignore_virtual=True)

    def sync_get_data(self, data_iterator, preprocess=None):
        """Every TP/CP rank of the end stages holds the same packed samples already; only the keys the middle
        stages need travel over PP."""
        from ..parallel.state import PM
        from ..utils.dist_utils import broadcast_tensors

        data = next(data_iterator) if self.is_data_source() and data_iterator is not None else None
        keys = self.global_data_keys
        if keys and PM.size_of("PP") > 1:
            sub = [type(data)] + [getattr(data, k, None) for k in keys] if data is not None and \
                PM.is_pipeline_first_stage(True) else None
            sub = broadcast_tensors(sub, src=PM.ranks_of("PP")[0], group=PM.group_of("PP"))
            if data is None:
                data = sub[0](**dict(zip(keys, sub[1:])))
        return data

    def preprocess_generated(self, data):
        from ..utils.general import recur_to

        if data is None:
            return data
        dev = "cuda" if torch.cuda.is_available() else "cpu"
        data = recur_to(data, dev)
        return {"input_ids": data.input_ids, "cu_seqlens": data.cu_seqlens, "max_seq_len": data.max_seq_len,
                "return_logits": True, "_samples": data}

    # ---------------------------------------------------------------------------- algorithm (overridable)
    def token_logprobs(self, data: PackedPPOSamples, logits: torch.Tensor, temperature: float = 1.0):
        """Log-probability of every label under vocab-sharded ``logits [S(/CP), V/TP]`` -> ``[S]`` (global)."""
        from ..ops.cross_entropy import vocab_parallel_cross_entropy
        from ..parallel.context_parallel import gather_from_balanced_cp_region, scatter_to_balanced_cp_region
        from ..parallel.state import PM

        labels = data.labels.reshape(-1).to(logits.device)
        if PM.size_of("CP") > 1:
            labels = scatter_to_balanced_cp_region(labels, dim=0)
        v_local = logits.shape[-1]
        if temperature != 1.0:
            logits = logits / temperature
        loss, _ = vocab_parallel_cross_entropy(logits, labels, PM.rank_in("TP") * v_local, PM.group_of("TP"))
        lp = -loss
        if PM.size_of("CP") > 1:
            lp = gather_from_balanced_cp_region(lp)
        return lp

    def get_advantage_and_returns(self, ragged_samples: PackedPPOSamples, ragged_values: torch.Tensor):
        """GAE over the response tokens of every sample; the (clipped) reward lands on the last one."""
        from ..utils.rl_utils import compute_gae

        mask = ragged_samples.is_gen_mask.reshape(-1).to(ragged_values.device).bool()
        values = ragged_values.reshape(-1)[mask].float()
        cu = ragged_samples.cu_seqlens.tolist()
        flat_mask = mask.cpu()
        lens = [int(flat_mask[b:e].sum()) for b, e in zip(cu[:-1], cu[1:])]
        cu_resp = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device=values.device)
        rewards = torch.zeros_like(values)
        ends = (cu_resp[1:] - 1).long()
        raw = torch.tensor([float(s.raw_reward) for s in ragged_samples.samples], device=values.device)
        raw = raw.clamp(-self.reward_clip, self.reward_clip)
        keep = torch.tensor([n > 0 for n in lens], device=values.device)
        rewards[ends[keep]] = raw[keep]
        if ragged_samples.ref_logprobs is not None and self.ref_kl_penalty_coeff and \
                ragged_samples.actor_logprobs is not None:
            kl = (ragged_samples.actor_logprobs - ragged_samples.ref_logprobs).to(values.device)
            rewards = rewards - self.ref_kl_penalty_coeff * kl
        adv, _ = compute_gae(values, rewards, self.ppo_actor_lambda, self.ppo_gae_gamma, cu_resp)
        _, ret = compute_gae(values, rewards, self.ppo_critic_lambda, self.ppo_gae_gamma, cu_resp)
        ragged_samples.advantages, ragged_samples.returns, ragged_samples.values = adv, ret, values
        return adv, ret

    def group_relative_advantages(self, ragged_samples: PackedPPOSamples):
        """Critic-free estimate: reward minus the mean over the rollouts of the same prompt, spread over the
        response tokens."""
        rewards = torch.tensor([float(s.raw_reward) for s in ragged_samples.samples])
        base = torch.tensor([float(getattr(s, "meta", {}).get("group_mean_reward", 0.0)) for s in ragged_samples.samples])
        mask = ragged_samples.is_gen_mask.reshape(-1).cpu()
        cu = ragged_samples.cu_seqlens.tolist()
        lens = [int(mask[b:e].sum()) for b, e in zip(cu[:-1], cu[1:])]
        adv = torch.cat([torch.full((n,), float(r - b)) for r, b, n in zip(rewards, base, lens)])
        ragged_samples.advantages = adv
        ragged_samples.returns = adv.clone()
        return adv, adv

    def actor_loss_func(self, data, outputs, loss_scale=1.0):
        from ..utils.metrics import GlobalMetrics

        samples: PackedPPOSamples = data["_samples"]
        mask = samples.is_gen_mask.reshape(-1).to(outputs.device).bool()
        new_lp = self.token_logprobs(samples, outputs, self.policy_actor_temperature)[mask]
        samples.actor_logprobs = new_lp.detach()
        old_lp = samples.logprobs.to(new_lp.device).float() if samples.logprobs is not None and \
            not self.use_offpolicy_without_is else new_lp.detach()
        adv = samples.advantages.to(new_lp.device).float().clamp(self.advantage_clip_min, self.advantage_clip_max)
        ratio = torch.exp(new_lp - old_lp)
        s1, s2 = ratio * adv, ratio.clamp(1 - self.ppo_clip, 1 + self.ppo_clip) * adv
        pg = -torch.minimum(s1, s2)
        if self.dual_clip_eps and self.dual_clip_eps > 1:
            pg = torch.where(adv < 0, torch.minimum(pg, -self.dual_clip_eps * adv), pg)
        loss = pg.mean()
        with torch.no_grad():
            low, high = (ratio < 1 - self.ppo_clip) & (adv < 0), (ratio > 1 + self.ppo_clip) & (adv > 0)
            GlobalMetrics.ppo_clip_frac.add(((ratio - 1).abs() > self.ppo_clip).float().mean())
            GlobalMetrics.ppo_clip_count.add((low | high).float().mean())     # tokens whose gradient the clip removed
            GlobalMetrics.ppo_lower_bound_clip_count.add(low.float().mean())
            GlobalMetrics.ppo_upper_bound_clip_count.add(high.float().mean())
            GlobalMetrics.ratio_diff.add((ratio - 1).abs().mean())
            # E_old[r log r]: KL(new || old) estimated on the old policy's samples
            GlobalMetrics.reverse_kl_with_sample_dist.add((ratio * (new_lp - old_lp)).mean())
        if samples.ref_logprobs is not None and self.ref_kl_loss_coeff > 0:
            kl = (new_lp - samples.ref_logprobs.to(new_lp.device)).mean()
            loss = loss + self.ref_kl_loss_coeff * kl
            GlobalMetrics.kl_with_ref_dist.add(kl.detach())
        if self.sample_kl_loss_coeff > 0:
            kl_old = (new_lp - old_lp).mean()
            loss = loss + self.sample_kl_loss_coeff * kl_old
            GlobalMetrics.kl_with_sample_dist.add(kl_old.detach())
        GlobalMetrics.ppo_loss.add(loss.detach())
        return loss * loss_scale

    def critic_loss_func(self, data, outputs, loss_scale=1.0):
        from ..parallel.context_parallel import gather_from_balanced_cp_region
        from ..parallel.state import PM
        from ..utils.metrics import GlobalMetrics

        samples: PackedPPOSamples = data["_samples"]
        values = outputs.reshape(outputs.shape[0], -1)[:, 0].float()
        if PM.size_of("CP") > 1:
            values = gather_from_balanced_cp_region(values)
        mask = samples.is_gen_mask.reshape(-1).to(values.device).bool()
        values = values[mask]
        target = samples.returns.to(values.device).float()
        if not self.critic_value_clip:
            # no clip range: the plain mean-squared error against the returns, which is what the reference's RLVR
            # experiment trains its critic with (playground/rlvr/qwen3_1p5b_rlvr_math.py:289-305)
            l1 = l2 = (values - target) ** 2
            loss = l1.mean()
        else:
            old = samples.values.to(values.device).float() if samples.values is not None else values.detach()
            clipped = old + (values - old).clamp(-self.critic_value_clip, self.critic_value_clip)
            l1, l2 = (values - target) ** 2, (clipped - target) ** 2
            loss = 0.5 * torch.maximum(l1, l2).mean()
        GlobalMetrics.value_clip_frac.add((l2 > l1).float().mean().detach())
        GlobalMetrics.ppo_value_clip_count.add((l2 > l1).float().mean().detach())
        GlobalMetrics.ppo_returns.add(target.mean().detach())
        GlobalMetrics.ppo_values.add(values.mean().detach())
        GlobalMetrics.critic_loss.add(loss.detach())
        return loss * loss_scale

    def batch_reward_function(self, samples: list) -> list:
        raise NotImplementedError

    def record(self, response: str, response_token: list, reward: float, sample: PPOSample):
        from ..text_processing.math_utils import repeatness_score
        from ..utils.metrics import GlobalMetrics

        rep = repeatness_score(response)
        GlobalMetrics.repeatness_score.add(rep)
        GlobalMetrics.repeatness_rate.add(float(rep > 0.2))
        lp = sample.logprobs.float().mean() if sample.logprobs is not None and len(sample.logprobs) else None
        if reward >= 0.5:
            GlobalMetrics.repeatness_rate_correct.add(float(rep > 0.2))
            if lp is not None:
                GlobalMetrics.rollout_logprob_correct.add(lp)
        else:
            GlobalMetrics.repeatness_rate_incorrect.add(float(rep > 0.2))
            if lp is not None:
                GlobalMetrics.rollout_logprob_incorrect.add(lp)

    def filter_samples(self, samples: list) -> list:
        from ..utils.metrics import GlobalMetrics

        GlobalMetrics.sample_filter_rate.add(0.0)
        return samples

    def log_generation_metrics(self, all_samples: list) -> None:
        from ..utils.metrics import GlobalMetrics

        if not all_samples:
            return
        n_gen = [int(s.is_gen_mask.sum()) for s in all_samples]
        GlobalMetrics.rollout_avg_tokens.add(sum(n_gen) / len(n_gen))
        GlobalMetrics.truncated_rate.add(
            sum(s.stop_type in (StopType.MAX_LEN, StopType.MAX_DECODE) for s in all_samples) / len(all_samples))
        lps = [s.logprobs.float().mean() for s in all_samples if s.logprobs is not None and len(s.logprobs)]
        if lps:
            GlobalMetrics.rollout_logprob.add(torch.stack(lps).mean())
        GlobalMetrics.rollout_samples.add(float(len(all_samples)))
        tokenizer = self.build_tokenizer() if callable(getattr(self, "build_tokenizer", None)) else None
        if tokenizer is not None:
            self.log_solution_think_tokens(all_samples, tokenizer)
        for s, n in zip(all_samples, n_gen):
            GlobalMetrics.rollout_tokens_hist.add(float(n))
            cut = float(s.stop_type in (StopType.MAX_LEN, StopType.MAX_DECODE))
            for tag in _sample_tags(s):
                GlobalMetrics.rollout_avg_tokens_grouped.add(float(n), subname=tag)
                GlobalMetrics.truncated_rate_grouped.add(cut, subname=tag)
                if s.logprobs is not None and len(s.logprobs):
                    GlobalMetrics.rollout_logprob_grouped.add(s.logprobs.float().mean(), subname=tag)

    def log_solution_think_tokens(self, all_samples: list, tokenizer) -> None:
        """Average generated tokens up to and including the first ``</think>`` token, and after it (a response
        without the marker is all solution).  The marker is looked up as a token id, nothing is decoded; a
        tokenizer that does not have it as one token fills neither metric.  Reference: exp/rl.py:700-740."""
        from ..text_processing.content_parsing import THINK_END_TOKEN
        from ..utils.metrics import GlobalMetrics

        ids = tokenizer.encode(THINK_END_TOKEN, add_special_tokens=False)
        if len(ids) != 1 or not all_samples:
            return
        think = solution = 0
        for s in all_samples:
            gen = torch.as_tensor(s.trajectory)[torch.as_tensor(s.is_gen_mask).bool()]
            hits = (gen == ids[0]).nonzero()
            cut = int(hits[0]) + 1 if hits.numel() else 0
            think += cut
            solution += gen.numel() - cut
        GlobalMetrics.rollout_avg_think_tokens.add(think / len(all_samples))
        GlobalMetrics.rollout_avg_solution_tokens.add(solution / len(all_samples))

    def log_reward_metrics(self, all_samples: list) -> None:
        from ..utils.metrics import GlobalMetrics

        if not all_samples:
            return
        r = torch.tensor([float(s.raw_reward) for s in all_samples])
        GlobalMetrics.reward_mean.add(r.mean())
        GlobalMetrics.reward_max.add(r.max())
        GlobalMetrics.reward_min.add(r.min())
        groups: dict = {}
        kind_of_prompt: dict = {}
        for s in all_samples:
            groups.setdefault(s.prompt_id, []).append(float(s.raw_reward))
            fn_tag, file_tag = _sample_tags(s)
            kind_of_prompt[s.prompt_id] = fn_tag
            for m in (GlobalMetrics.reward_func_mean, GlobalMetrics.reward_func_max, GlobalMetrics.reward_func_min):
                m.add(float(s.raw_reward), subname=fn_tag)
            for m in (GlobalMetrics.reward_filename_mean, GlobalMetrics.reward_filename_max, GlobalMetrics.reward_filename_min):
                m.add(float(s.raw_reward), subname=file_tag)
        for s in all_samples:
            g = groups[s.prompt_id]
            if s.meta is None:
                s.meta = {}
            s.meta["group_mean_reward"] = sum(g) / len(g)
        kinds = {"all_correct": 0, "all_fail": 0, "some_correct": 0}
        for pid, g in groups.items():
            ok = sum(x >= 0.5 for x in g)
            kind = "all_correct" if ok == len(g) else "all_fail" if ok == 0 else "some_correct"
            kinds[kind] += 1
            GlobalMetrics.correctness_subclass.add(1.0, subname=f"{kind}/{kind_of_prompt[pid]}")
        for k, v in kinds.items():
            GlobalMetrics.correctness.add(float(v), subname=k)

    def log_sampling_logprob_metrics(self, samples: list) -> None:
        from ..utils.metrics import GlobalMetrics

        diffs = [(s.actor_logprobs.float().cpu() - s.logprobs.float().cpu()).abs() for s in samples
                 if s.actor_logprobs is not None and s.logprobs is not None and len(s.logprobs)]
        if diffs:
            d = torch.cat(diffs)
            GlobalMetrics.logprob_diff_mean.add(d.mean())
            GlobalMetrics.logprob_diff_max.add(d.max())
            GlobalMetrics.sampling_logprob_diff.add(torch.stack([x.mean() for x in diffs]).mean())   # mean over samples
            GlobalMetrics.sampling_logprob_diff_max.add(d.max())
            pairs = [(s.actor_logprobs.float().cpu(), s.logprobs.float().cpu()) for s in samples
                     if s.actor_logprobs is not None and s.logprobs is not None and len(s.logprobs)]
            new, old = torch.cat([a for a, _ in pairs]), torch.cat([b for _, b in pairs])
            for metric, data in ((GlobalMetrics.sampling_logprob_diff_quantile, d),
                                 (GlobalMetrics.sampling_ratio_diff, (torch.exp(new - old) - 1).abs()),
                                 (GlobalMetrics.ratio_diff_quantile, torch.exp(new - old) - 1),
                                 (GlobalMetrics.new_logprob, new), (GlobalMetrics.old_logprob, old),
                                 (GlobalMetrics.new_prob, new.exp()), (GlobalMetrics.old_prob, old.exp())):
                for tag, value in quantile_summary(data).items():
                    metric.add(value, subname=tag)


def _sample_tags(sample) -> tuple[str, str]:
    """``(reward function, data file)`` a sample's prompt belongs to, from its ground truth (``"default"`` /
    ``"unknown"`` when the data does not say), the two keys the grouped rollout metrics are kept under."""
    gt = sample.ground_truth if isinstance(getattr(sample, "ground_truth", None), dict) else {}
    path = str(gt.get("file_path", "unknown"))
    return str(gt.get("reward_fn_type", "default")), os.path.basename(path).split(".")[0] or "unknown"


def quantile_summary(data: torch.Tensor, max_elems: int = 200000) -> dict:
    """``min / max`` of all entries and ``q01 q05 q10 q90 q95 q99`` of a random tenth of them (at most ``max_elems``;
    quantiles of a million token log-probabilities per step would cost more than they tell)."""
    flat = data.detach().float().flatten().cpu()
    take = max(min(flat.numel() // 10, max_elems), 1)
    picked = flat[torch.randperm(flat.numel())[:take]]
    q = torch.quantile(picked, torch.tensor([0.01, 0.05, 0.1, 0.9, 0.95, 0.99]))
    return {"min": flat.min(), "max": flat.max(), **dict(zip(("q01", "q05", "q10", "q90", "q95", "q99"), q))}


class PPOLikeExp(BaseExp):
    data_cfg: DataConfig = DataConfig
    actor_model_cfg: ActorModelConfig = ActorModelConfig
    actor_scheduler_cfg: SchedulerConfig = SchedulerConfig
    actor_grad_manager_cfg: GradientManagerConfig = GradientManagerConfig
    critic_model_cfg: CriticModelConfig | None = None
    critic_scheduler_cfg: SchedulerConfig | None = None
    critic_grad_manager_cfg: GradientManagerConfig | None = None
    checkpoint_cfg: PPOCheckpointCfg = PPOCheckpointCfg
    trainer_cfg: PPOLikeTrainerConfig = PPOLikeTrainerConfig
    metric_cfg: PPOMetricConfig = PPOMetricConfig
    profiler_cfg: ProfilerConfig = ProfilerConfig

    def train(self):
        self.update_from_args()
        self.sanity_check()
        trainer = self.trainer_cfg.get_trainer_cls()(self)
        self.configure_optimizable()
        trainer.train()
        return trainer

    def configure_optimizable(self) -> None:
        """Hook between building the trainer and training: an experiment selects operator back-ends here with
        ``utils.optimizable.set_optimization``."""
