"""The standard evaluation set for a Step-3.5 checkpoint: expert-parallel vLLM servers over a whole node,
reasoning parser on (reference ``playground/eval/step3p5/step3p5_eval_simple_benchmarks.py``)."""
import os

from playground.eval.qwen3.qwen3_eval_simple_benchmarks import Exp as Qwen3EvalExp
from steptronoss_b200.exp.inference import VLLMDeployConfig


class Step3p5EvalVLLMDeployConfig(VLLMDeployConfig):
    def __init__(self):
        super().__init__()
        self.model_config_path = os.environ.get("STB200_EVAL_MODEL", "/models/Step-3.5-Flash")
        self.max_seq_len = 131072
        self.vllm_gpu_memory_utilization = 0.9
        self.vllm_tp, self.vllm_dp = 8, 1
        self.enable_expert_parallel = True
        self.enable_reasoning = True
        self.reasoning_parser = "deepseek_r1"
        self.max_cache_size = 128


class Exp(Qwen3EvalExp):
    vllm_cfg = Step3p5EvalVLLMDeployConfig

    def __init__(self):
        super().__init__()
        self.resource_cfg.vllm_replica = 1


if __name__ == "__main__":
    Exp().entrypoint()
