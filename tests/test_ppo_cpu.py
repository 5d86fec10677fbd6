"""PPO trainer end to end on CPU: fake in-process generation feeds the flow controller, the reference / actor /
critic passes fill log-probabilities and values, both models take optimizer steps, and the job checkpoints."""
import asyncio
import os
import random

import pytest
import torch

from steptronoss_b200.data.nextable import Nextable
from steptronoss_b200.exp.base_exp import DataConfig, GradientManagerConfig, ProfilerConfig
from steptronoss_b200.exp.lr_schedulers import ConstantSchedulerConfig
from steptronoss_b200.exp.rl import (ActorModelConfig, CriticModelConfig, EnvTrajectory, FlowControllerConfig,
                                     PackedPPOSamples, PPOCheckpointCfg, PPOLikeExp, PPOLikeTrainerConfig,
                                     PPOMetricConfig, PPOSample)
from steptronoss_b200.generation.async_generation import SingleGenerationController
from steptronoss_b200.generation.base_generatable import TrainableItem
from steptronoss_b200.generators.flow_controller import SimpleFlowController
from steptronoss_b200.models.common.parallel_embedding import OneDimensionalOutputEmbedding, OutputEmbeddingConfig
from steptronoss_b200.models.decoder_model import DecoderLLMConfig

VOCAB = 64


class FakeRollout(TrainableItem):
    def __init__(self, idx):
        super().__init__()
        self.idx = idx

    async def generate(self):
        return self.idx

    async def generate_for_train(self):
        await asyncio.sleep(0)
        rnd = random.Random(self.idx)
        out = []
        for k in range(2):
            p, g = rnd.randint(3, 6), rnd.randint(4, 9)
            toks = [rnd.randrange(VOCAB) for _ in range(p + g)]
            # reward: fraction of even tokens in the response (something a policy can learn)
            r = sum(t % 2 == 0 for t in toks[p:]) / g
            out.append(EnvTrajectory(trajectory=toks, is_gen_mask=[0] * p + [1] * g, raw_reward=r,
                                     logprobs=[-3.0] * g,
                                     meta={"idx": self.idx, "ground_truth": {"reward_fn_type": "parity",
                                                                             "file_path": "/data/evens.jsonl"}}))
        return out


class Prompts(Nextable):
    def __init__(self):
        self.i = 0

    def __iter__(self):
        return self

    def __next__(self):
        self.i += 1
        return FakeRollout(self.i - 1)

    def state_dict(self):
        return {"i": self.i}

    def load_state_dict(self, sd):
        self.i = sd["i"]


class PromptData(DataConfig):
    def build_dataloader(self, dp_rank=0, dp_size=1):
        return Prompts()


class ValueHead(OutputEmbeddingConfig):
    def build_model(self, tied_embedding_weight=None):
        return OneDimensionalOutputEmbedding(self)


class Actor(ActorModelConfig, DecoderLLMConfig):
    pass


class Critic(CriticModelConfig, DecoderLLMConfig):
    out_embed_cfg = ValueHead


class Flow(FlowControllerConfig):
    def build_flow_controller(self):
        return SimpleFlowController(self, generator=SingleGenerationController(), deploy_fn=lambda models: None)


class Trainer(PPOLikeTrainerConfig):
    flow_cfg = Flow


class Exp(PPOLikeExp):
    data_cfg = PromptData
    actor_model_cfg = Actor
    critic_model_cfg = Critic
    actor_grad_manager_cfg = GradientManagerConfig
    critic_grad_manager_cfg = GradientManagerConfig
    actor_scheduler_cfg = ConstantSchedulerConfig
    critic_scheduler_cfg = ConstantSchedulerConfig
    checkpoint_cfg = PPOCheckpointCfg
    trainer_cfg = Trainer
    metric_cfg = PPOMetricConfig
    profiler_cfg = ProfilerConfig


def _fill_model(m, hidden=32):
    m.num_layers, m.hidden_size, m.params_dtype, m.variable_seq_lengths = 2, hidden, torch.float32, True
    a = m.attn_cfg
    a.num_attention_heads, a.num_attention_groups, a.head_dim, a.hidden_size = 2, 1, 16, hidden
    m.ffn_cfg.hidden_size, m.ffn_cfg.ffn_hidden_size = hidden, 64
    m.tok_embed_cfg.vocab_size = m.out_embed_cfg.vocab_size = VOCAB
    m.tok_embed_cfg.hidden_size = m.out_embed_cfg.hidden_size = hidden
    m.parallel_cfg.expert_tensor_parallel_size = 1


def _exp(tmp_path, use_critic=True):
    e = Exp()
    _fill_model(e.actor_model_cfg)
    _fill_model(e.critic_model_cfg)
    t = e.trainer_cfg
    t.train_iters, t.global_seq_length, t.global_batch_size, t.writer_backend = 3, 64, 1, []
    t.critic_warmup_iters, t.fix_iters, t.use_critic = 0, 2, use_critic
    t.flow_cfg.prompt_per_iter, t.flow_cfg.async_strategy = 6, "on-policy"
    for s in (e.actor_scheduler_cfg, e.critic_scheduler_cfg):
        s.lr, s.weight_decay, s.warmup_schedule = 1e-3, 0.0, 0
    e.checkpoint_cfg.save_dir = str(tmp_path)
    e.checkpoint_cfg.save_interval = 2
    e.checkpoint_cfg.async_save = False
    if not use_critic:
        e.critic_model_cfg = None
    return e


def test_packed_samples_layout():
    s = [PPOSample(trajectory=torch.arange(5), is_gen_mask=torch.tensor([0, 0, 1, 1, 1]).bool(),
                   logprobs=torch.zeros(3), raw_reward=1.0, meta={}),
         PPOSample(trajectory=torch.arange(4), is_gen_mask=torch.tensor([0, 1, 1, 1]).bool(),
                   logprobs=torch.zeros(3), raw_reward=0.0, meta={})]
    p = PackedPPOSamples.from_samples(s)
    assert p.input_ids.shape == (1, 10) and p.cu_seqlens.tolist() == [0, 5, 10] and p.cu_valid_sizes.tolist() == [0, 5, 9]
    assert p.labels[0, :9].tolist() == [1, 2, 3, 4, 0, 1, 2, 3, 0]
    # label-aligned mask: position t is trained when token t+1 was generated
    assert p.is_gen_mask[0].tolist() == [False, True, True, True, False, True, True, True, False, False]
    assert int(p.is_gen_mask.sum()) == p.logprobs.numel()


@pytest.mark.parametrize("use_critic", [True, False])
def test_ppo_trains_and_checkpoints(tmp_path, use_critic):
    exp = _exp(tmp_path, use_critic)
    exp.sanity_check()
    tr = exp.trainer_cfg.get_trainer_cls()(exp)
    tr.before_train()
    before = {n: p.detach().clone() for n, p in tr.actor.models.named_parameters()}
    tr.train_loop()
    assert tr.iteration == 3 and tr.actor_iteration >= 3
    moved = sum(float((p.detach() - before[n]).abs().sum()) for n, p in tr.actor.models.named_parameters())
    assert moved > 0
    keys = tr.history[-1]
    assert "reward_mean" in keys and "ppo_loss" in keys and (not use_critic or "critic_loss" in keys)
    # grouped by the prompt's reward function and data file, and the off-policy quantile groups
    for key in ("reward_func_max/parity", "reward_filename_mean/evens", "rollout_avg_tokens_grouped/parity",
                "truncated_rate_grouped/evens", "correctness_subclass/some_correct/parity", "new_logprob/q90",
                "sampling_ratio_diff/max", "ppo_clip_count", "ratio_diff", "rollout_samples"):
        assert key in keys, key
    assert float(keys["reward_func_min/parity"]) <= float(keys["reward_func_mean/parity"]) <= float(keys["reward_func_max/parity"])
    assert float(keys["old_logprob/min"]) == pytest.approx(-3.0) and float(keys["rollout_samples"]) == 12.0
    assert (not use_critic) or "ppo_values" in keys
    it_dir = os.path.join(exp.checkpoint_cfg.save_path, "it2")
    assert os.path.isdir(os.path.join(it_dir, "actor")) and os.path.exists(os.path.join(it_dir, "data.pkl"))
    assert os.path.isdir(os.path.join(it_dir, "critic")) == use_critic
    assert open(os.path.join(exp.checkpoint_cfg.save_path, "latest_ckpt")).read().strip() == it_dir


def test_get_normalizer_values_and_non_finite_inputs():
    import pytest
    import torch

    from steptronoss_b200.trainers.ppo_trainer import get_normalizer

    m, s = get_normalizer(torch.tensor([1.0, 2.0, 3.0, 4.0, 5.0]))
    assert torch.isclose(m, torch.tensor(3.0)) and torch.isclose(s, torch.tensor(2.0).sqrt())
    m, s = get_normalizer(torch.full((3,), 5.0))
    assert float(m) == 5.0 and float(s) == 0.0
    for bad in (float("nan"), float("inf")):
        with pytest.raises(ValueError, match="non-finite"):
            get_normalizer(torch.tensor([1.0, bad, 3.0]))


def test_evaluation_schedule_and_score_logging():
    import types

    from steptronoss_b200.trainers.ppo_trainer import PPOTrainer

    logged = []
    writer = types.SimpleNamespace(add_scalar=lambda k, v, it: logged.append((k, v, it)))
    evals = []
    eval_cfg = types.SimpleNamespace(eval=lambda: (evals.append(1), {"AIME2025": {"metric": {"score_avg": 0.25, "by": {"x": 1}}}})[1])
    tr = types.SimpleNamespace(ppo_cfg=types.SimpleNamespace(eval_interval=2, skip_first_eval=True),
                               exp=types.SimpleNamespace(eval_cfg=eval_cfg), iteration=0, writer=writer)
    due = []
    for it in range(5):
        tr.iteration = it
        due.append(PPOTrainer.eval_due(tr))
    assert due == [False, False, True, False, True]
    tr.ppo_cfg.skip_first_eval, tr.iteration = False, 0
    assert PPOTrainer.eval_due(tr)
    tr.exp.eval_cfg = None
    assert not PPOTrainer.eval_due(tr)
    tr.exp.eval_cfg, tr.iteration = eval_cfg, 4
    summary = PPOTrainer.eval(tr)
    assert evals == [1] and summary["AIME2025"]["metric"]["score_avg"] == 0.25
    assert logged == [("eval/AIME2025/score_avg", 0.25, 4)]


def test_quantile_summary_and_sample_tags():
    from steptronoss_b200.exp.rl import _sample_tags, quantile_summary

    torch.manual_seed(0)
    q = quantile_summary(torch.arange(1000.0))
    assert float(q["min"]) == 0.0 and float(q["max"]) == 999.0
    assert float(q["q01"]) <= float(q["q10"]) <= float(q["q90"]) <= float(q["q99"]) and 700 < float(q["q90"])
    assert set(quantile_summary(torch.tensor([2.0]))) == {"min", "max", "q01", "q05", "q10", "q90", "q95", "q99"}
    s = PPOSample()
    assert _sample_tags(s) == ("default", "unknown")
    s.ground_truth = {"reward_fn_type": "math", "file_path": "s3://bucket/train/gsm8k.v2.jsonl"}
    assert _sample_tags(s) == ("math", "gsm8k")


def test_think_and_solution_token_split():
    from steptronoss_b200.utils.metrics import GlobalMetrics, Metric

    class Tok:
        def __init__(self, ids):
            self.ids = ids

        def encode(self, text, add_special_tokens=False):
            return self.ids

    GlobalMetrics.clear()
    GlobalMetrics.register("rollout_avg_think_tokens", Metric().mean("time"))
    GlobalMetrics.register("rollout_avg_solution_tokens", Metric().mean("time"))
    cfg = PPOLikeTrainerConfig()
    a = PPOSample(trajectory=torch.tensor([5, 5, 9, 7, 60, 3, 3]), is_gen_mask=torch.tensor([0, 0, 1, 1, 1, 1, 1]))
    b = PPOSample(trajectory=torch.tensor([5, 1, 2, 3]), is_gen_mask=torch.tensor([0, 1, 1, 1]))        # no marker
    cfg.log_solution_think_tokens([a, b], Tok([60]))
    out = GlobalMetrics.reduce_all()
    assert float(out["rollout_avg_think_tokens"]) == 1.5 and float(out["rollout_avg_solution_tokens"]) == 2.5
    cfg.log_solution_think_tokens([a, b], Tok([60, 61]))                   # the marker is not one token: nothing logged
    assert GlobalMetrics.rollout_avg_think_tokens.values == []
    GlobalMetrics.clear()


def test_ppo_auto_resume_takes_every_role_from_the_latest_checkpoint(tmp_path):
    exp = _exp(tmp_path, True)
    exp.sanity_check()
    tr = exp.trainer_cfg.get_trainer_cls()(exp)
    tr.before_train()
    tr.train_loop()                                                    # writes it2 (interval 2 of 3 iterations)
    trained = {n: p.detach().clone() for n, p in tr.actor.models.named_parameters()}
    again = _exp(tmp_path, True)
    again.checkpoint_cfg.actor.load_option.none(but=["model"])         # how the job was told to START
    again.checkpoint_cfg.actor.load_safetensors = "/models/pretrained"
    again.sanity_check()
    tr2 = again.trainer_cfg.get_trainer_cls()(again)
    tr2.before_train()
    ck = again.checkpoint_cfg
    assert ck.load_path.endswith("it2") and ck.actor.load_path.endswith(os.path.join("it2", "actor"))
    assert ck.actor.load_option.optimizer and ck.actor.load_safetensors is None and ck.critic.load_path.endswith("critic")
    assert all(os.path.isdir(r.load_path) for r in (ck.actor, ck.critic, ck.reference) if r.load_path)
    assert tr2.actor_iteration > 0
    first = next(iter(trained))
    # the parameters are those of iteration 2, not of a fresh initialisation and not those after iteration 3
    fresh = _exp(tmp_path / "other", True)
    fresh.sanity_check()
    tr3 = fresh.trainer_cfg.get_trainer_cls()(fresh)
    tr3.before_train()
    p2, p3 = dict(tr2.actor.models.named_parameters())[first], dict(tr3.actor.models.named_parameters())[first]
    assert not torch.equal(p2, p3)


def test_critic_loss_is_plain_mse_without_a_clip_range():
    from steptronoss_b200.utils.metrics import GlobalMetrics

    GlobalMetrics.clear()
    cfg = PPOLikeTrainerConfig()
    s = PackedPPOSamples()
    s.is_gen_mask = torch.tensor([[0, 1, 1, 1]]).bool()
    s.returns, s.values = torch.tensor([1.0, 0.0, 2.0]), torch.tensor([0.9, 0.0, 0.0])
    out = torch.tensor([[5.0], [1.5], [0.0], [1.0]])                       # the value of the prompt token is not trained
    cfg.critic_value_clip = None
    assert float(cfg.critic_loss_func({"_samples": s}, out)) == pytest.approx(float(((torch.tensor([1.5, 0.0, 1.0]) - s.returns) ** 2).mean()))
    cfg.critic_value_clip = 0.2
    # clipped: values may move 0.2 from the sampling pass; the worse of the two errors counts, halved
    clipped = torch.tensor([0.9 + 0.2, 0.0, 0.2])
    want = 0.5 * torch.maximum((torch.tensor([1.5, 0.0, 1.0]) - s.returns) ** 2, (clipped - s.returns) ** 2).mean()
    assert float(cfg.critic_loss_func({"_samples": s}, out)) == pytest.approx(float(want))
    from playground.rlvr.qwen3_1p5b_rlvr_math import RLVRTrainerConfig

    assert RLVRTrainerConfig().critic_value_clip is None
