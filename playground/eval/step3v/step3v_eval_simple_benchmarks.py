"""IFBench on a Step3-VL checkpoint, sampled the way the model's report does it: four answers per prompt at
temperature 1.0, top-p 1.0, no top-k, 64k context; scores are fractions (0.43 = 43 %), with pass@1/2/4 beside the
loose and strict accuracies (reference ``playground/eval/step3v/step3v_eval_simple_benchmarks.py``).  One GPU is
enough for the 10B model: one vLLM task, eager mode.

    python -m steptronoss_b200.launch.mp_run playground/eval/step3v/step3v_eval_simple_benchmarks.py \\
        vllm_cfg.model_config_path=/models/Step3-VL-10B eval_cfg.datasets_dir=/data/simple_benchmarks

Setting ``eval_cfg.selected_datasets`` to other names runs those benchmarks with the standard settings.
"""
import os

from playground.eval.qwen3.qwen3_eval_simple_benchmarks import EvalResourceConfig, EvalTokenizerConfig
from playground.eval.qwen3.qwen3_eval_simple_benchmarks import Exp as Qwen3EvalExp
from playground.eval.eval_sets.simple_eval import SimpleBenchmarksEvalConfig
from steptronoss_b200.exp.inference import VLLMDeployConfig


class Step3VEvalResourceConfig(EvalResourceConfig):
    vllm_replica: int = 1

    def __init__(self):
        super().__init__()
        self.gpu = 1
        self.vllm_replica = 1
        self.sync_task_specs()


class Step3VEvalVLLMDeployConfig(VLLMDeployConfig):
    def __init__(self):
        super().__init__()
        self.model_config_path = os.environ.get("STB200_EVAL_MODEL", "/models/Step3-VL-10B")
        self.max_seq_len = 65536
        self.vllm_gpu_memory_utilization = 0.85
        self.vllm_tp, self.vllm_dp = 1, 1
        self.reasoning_parser = "deepseek_r1"
        self.toolcall_parser = "hermes"
        self.vllm_enable_chunked_prefill = True
        self.vllm_enable_prefix_caching = True
        self.vllm_enforce_eager = True
        self.vllm_max_num_batched_tokens = 8192
        self.max_cache_size = 64


class Step3VSimpleBenchmarksEvalConfig(SimpleBenchmarksEvalConfig):
    tokenizer_cfg = EvalTokenizerConfig
    selected_datasets = "IFBENCH"
    chat_template_args = {}
    num_concurrent_requests = 8
    max_decode_steps = 65536
    ifbench_sample_per_prompt: int = 4
    ifbench_temperature: float = 1.0
    ifbench_top_p: float = 1.0
    ifbench_top_k: int = 0
    """0 switches top-k off in vLLM"""

    def build_benchmarks(self) -> list:
        self.sample_per_prompt = dict(self.sample_per_prompt) | {"IFBENCH": self.ifbench_sample_per_prompt}
        self.benchmark_options = dict(self.benchmark_options) | {"IFBENCH": {"sampling_params": {
            "temperature": self.ifbench_temperature, "top_p": self.ifbench_top_p, "top_k": self.ifbench_top_k}}}
        return super().build_benchmarks()


class Exp(Qwen3EvalExp):
    vllm_cfg = Step3VEvalVLLMDeployConfig
    resource_cfg = Step3VEvalResourceConfig
    eval_cfg = Step3VSimpleBenchmarksEvalConfig


if __name__ == "__main__":
    Exp().entrypoint()
