"""RLVR on boxed-answer math with a Qwen3-1.7B actor and critic (reference
``playground/rlvr/qwen3_1p5b_rlvr_math.py``).

One node, three roles started by ``python -m steptronoss_b200.launch.mp_run`` (or one task per role on a
cluster): ``trainer`` (GPUs 0-3, actor + critic + frozen reference with role swapping), ``generator`` (GPUs 4-7,
one vLLM server behind the router, weights refreshed from the trainer after every step) and ``router`` (CPU).
Prompts come from ``data_cfg.prompt_file`` (jsonl with ``prompt`` / ``answer``) or, without a file, a single
built-in question, which is enough to watch the reward rise.

    python -m steptronoss_b200.launch.mp_run playground/rlvr/qwen3_1p5b_rlvr_math.py tokenizer_cfg.tokenizer_path=/models/Qwen3-1.7B
"""
import json
import os

from playground.pretrain.qwen3.qwen3_1p7b import Qwen3_1p7BConfig, Qwen3_1p7BOutputEmbeddingConfig
from playground.rlvr.simple_trainable import SimpleTrainable
from steptronoss_b200.config import Ref
from steptronoss_b200.data.nextable import Nextable
from steptronoss_b200.exp.base_exp import DataConfig, GradientManagerConfig, ProfilerConfig, TokenizerConfig
from steptronoss_b200.exp.inference import VLLMDeployConfig
from steptronoss_b200.exp.lr_schedulers import ConstantSchedulerConfig
from steptronoss_b200.exp.optimizer import AdamConfig
from steptronoss_b200.exp.resources import ResourceConfig, TaskSpec
from steptronoss_b200.exp.rl import (ActorModelConfig, CriticModelConfig, FlowControllerConfig, PPOCheckpointCfg,
                                     PPOLikeExp, PPOLikeTrainerConfig, PPOMetricConfig)
from steptronoss_b200.generation.base_generatable import EndpointGetter, ModelNameGetter
from steptronoss_b200.generation.vllm.vllm_router import VLLMRouterConfig

MODEL_DIR = os.environ.get("STB200_QWEN3_1P7B", "/models/Qwen3-1.7B")
BUILTIN_PROMPTS = [{"prompt": "How many times does the letter r occur in the word strawberry? "
                              "Give the final answer as \\boxed{...}.", "answer": "3"}]


class PromptStream(Nextable):
    """Endless stream of rollout items over a list of ``{prompt, answer}`` records (resumable by position)."""

    def __init__(self, records, render, endpoint_getter, model_name_getter, max_tokens, dp_rank=0, dp_size=1):
        super().__init__()
        self.records, self.render = records, render
        self.endpoint_getter, self.model_name_getter, self.max_tokens = endpoint_getter, model_name_getter, max_tokens
        self.pos, self.stride = dp_rank, dp_size

    def __next__(self):
        rec = self.records[self.pos % len(self.records)]
        self.pos += self.stride
        return SimpleTrainable(self.render(rec["prompt"]), str(rec["answer"]), self.endpoint_getter,
                               self.model_name_getter, max_tokens=self.max_tokens)

    def state_dict(self):
        return {"pos": self.pos}

    def load_state_dict(self, sd):
        self.pos = sd["pos"]


class MathPromptDataConfig(DataConfig):
    prompt_file: str | None = None
    prompt_key: str = "prompt"
    answer_key: str = "answer"
    max_tokens: int = 1024
    build_tokenizer = Ref("..tokenizer_cfg.build_tokenizer")
    vllm_cfg = Ref("..actor_model_cfg.vllm_cfg")

    def load_records(self) -> list:
        if not self.prompt_file:
            return list(BUILTIN_PROMPTS)
        with open(self.prompt_file, encoding="utf-8") as f:
            rows = [json.loads(line) for line in f if line.strip()]
        return [{"prompt": r[self.prompt_key], "answer": r[self.answer_key]} for r in rows]

    def build_dataloader(self, dp_rank=0, dp_size=1):
        tok = self.build_tokenizer()

        def render(question: str) -> str:
            return tok.apply_chat_template([{"role": "user", "content": question}], tokenize=False,
                                           add_generation_prompt=True)

        v = self.vllm_cfg
        return PromptStream(self.load_records(), render, EndpointGetter(v.router_addr_key),
                            ModelNameGetter(v.model_name_template), self.max_tokens, dp_rank, dp_size)


class Qwen3TokenizerConfig(TokenizerConfig):
    tokenizer_path: str = MODEL_DIR


class RLVRResourceConfig(ResourceConfig):
    def __init__(self):
        super().__init__()
        self.replica, self.gpu, self.node_type = 1, 4, "gpu"
        self.task_specs = {
            "trainer": TaskSpec(envs={"ROLE": "trainer", "CUDA_VISIBLE_DEVICES": "0,1,2,3"}, is_critical=True,
                                command="{TORCHRUN} {COMMAND}"),
            "generator": TaskSpec(envs={"ROLE": "generator", "CUDA_VISIBLE_DEVICES": "4,5,6,7"}),
            "router": TaskSpec(gpu=0, node_type="cpu", envs={"ROLE": "router"}),
        }


class RLVRVLLMDeployConfig(VLLMDeployConfig):
    def __init__(self):
        super().__init__()
        self.model_config_path = MODEL_DIR
        self.max_seq_len = 40960
        self.model_name_template = "deployed-model-{EXP_ID}"
        self.vllm_tp = 4
        self.hot_path = os.environ.get("STB200_HOT_PATH", "/dev/shm/stb200_hot")


class RLVRActorModelConfig(ActorModelConfig, Qwen3_1p7BConfig):
    vllm_cfg = RLVRVLLMDeployConfig


class ValueHeadConfig(Qwen3_1p7BOutputEmbeddingConfig):
    def build_model(self, tied_embedding_weight=None):
        import torch

        from steptronoss_b200.models.common.parallel_embedding import OneDimensionalOutputEmbedding

        head = OneDimensionalOutputEmbedding(self)
        torch.nn.init.trunc_normal_(head.output.weight, std=1e-5)   # values start at zero
        return head


class RLVRCriticModelConfig(CriticModelConfig, Qwen3_1p7BConfig):
    out_embed_cfg = ValueHeadConfig

    def __init__(self):
        super().__init__()
        self.tie_embedding = False


class ActorGradManagerConfig(GradientManagerConfig):
    optimizer_cfg = AdamConfig

    def __init__(self):
        super().__init__()
        self.optimizer_cfg.lr = Ref("...actor_scheduler_cfg.lr")
        self.optimizer_cfg.weight_decay = Ref("...actor_scheduler_cfg.weight_decay")


class CriticGradManagerConfig(GradientManagerConfig):
    optimizer_cfg = AdamConfig

    def __init__(self):
        super().__init__()
        self.optimizer_cfg.lr = Ref("...critic_scheduler_cfg.lr")
        self.optimizer_cfg.weight_decay = Ref("...critic_scheduler_cfg.weight_decay")


class OnPolicyFlowControllerConfig(FlowControllerConfig):
    def __init__(self):
        super().__init__()
        self.async_strategy = "on-policy"
        self.prompt_per_iter = 64


class RLVRTrainerConfig(PPOLikeTrainerConfig):
    """GAE over the response tokens with the outcome reward on the last one and the clipped surrogate are the trainer
    configuration's defaults; the critic regresses on the returns with a plain mean-squared error, as in the reference's
    experiment of the same name."""

    flow_cfg = OnPolicyFlowControllerConfig
    critic_value_clip = None


class Exp(PPOLikeExp):
    resource_cfg = RLVRResourceConfig
    vllm_router_cfg: VLLMRouterConfig = VLLMRouterConfig
    tokenizer_cfg = Qwen3TokenizerConfig
    data_cfg = MathPromptDataConfig
    actor_model_cfg = RLVRActorModelConfig
    critic_model_cfg = RLVRCriticModelConfig
    actor_grad_manager_cfg = ActorGradManagerConfig
    actor_scheduler_cfg = ConstantSchedulerConfig
    critic_grad_manager_cfg = CriticGradManagerConfig
    critic_scheduler_cfg = ConstantSchedulerConfig
    checkpoint_cfg = PPOCheckpointCfg
    trainer_cfg = RLVRTrainerConfig
    metric_cfg = PPOMetricConfig
    profiler_cfg = ProfilerConfig

    def __init__(self):
        super().__init__()
        self.log_dir = "./tensorboard_logs"
        t = self.trainer_cfg
        t.train_iters = 1000
        t.global_seq_length = 4096
        t.fix_iters = 1
        t.fix_iters_critic = 1
        for m in (self.actor_model_cfg, self.critic_model_cfg):
            m.parallel_cfg.tensor_model_parallel_size = 4
        self.actor_scheduler_cfg.lr = 1e-6
        self.critic_scheduler_cfg.lr = 5e-6
        c = self.checkpoint_cfg
        c.actor.load_safetensors = MODEL_DIR
        c.critic.load_safetensors = MODEL_DIR
        c.critic.strict_load_model = False      # the value head is new
        c.reference.load_safetensors = MODEL_DIR
        c.save_dir = "./checkpoints"
        c.save_interval = 50

    def entrypoint(self):
        role = os.environ.get("ROLE", "trainer")
        if role == "router":
            self.vllm_router_cfg.run()
        elif role == "generator":
            self.actor_model_cfg.vllm_cfg.run_as_worker()
        elif role == "trainer":
            self.train()
        else:
            raise ValueError(f"unknown ROLE: {role}")


if __name__ == "__main__":
    Exp().entrypoint()
