"""Evaluate a Qwen3 checkpoint on the standard set (reference
``playground/eval/qwen3/qwen3_1p7b_eval_simple_benchmarks.py``).  Roles: ``evaluator`` (CPU; waits for the
servers, runs the benchmarks), ``vllm`` x ``resource_cfg.vllm_replica`` (one server per task, data-parallel over
the node's 8 GPUs) and ``router`` (CPU).

    python -m steptronoss_b200.launch.mp_run playground/eval/qwen3/qwen3_eval_simple_benchmarks.py \\
        vllm_cfg.model_config_path=/models/Qwen3-8B eval_cfg.datasets_dir=/data/simple_benchmarks
"""
import os

from playground.eval.eval_sets.simple_eval import SimpleBenchmarksEvalConfig
from steptronoss_b200.config import Ref
from steptronoss_b200.exp.base_exp import BaseExp, TokenizerConfig
from steptronoss_b200.exp.inference import VLLMDeployConfig
from steptronoss_b200.exp.resources import ResourceConfig, TaskSpec
from steptronoss_b200.generation.vllm.vllm_router import VLLMRouterConfig
from steptronoss_b200.utils.logger import logger


class EvalResourceConfig(ResourceConfig):
    vllm_replica: int = 2

    def __init__(self):
        super().__init__()
        self.command = "python {COMMAND}"
        self.replica, self.gpu, self.node_type = 1, 8, "gpu"
        self.sync_task_specs()

    def sync_task_specs(self) -> None:
        self.task_specs = {
            "evaluator": TaskSpec(gpu=0, node_type="cpu", envs={"ROLE": "evaluator"}, is_critical=True),
            "vllm": TaskSpec(replica=self.vllm_replica, envs={"ROLE": "vllm"}),
            "router": TaskSpec(gpu=0, node_type="cpu", envs={"ROLE": "router"}),
        }

    def find_leaf_task_specs(self):
        self.sync_task_specs()
        return super().find_leaf_task_specs()


class Qwen3EvalVLLMDeployConfig(VLLMDeployConfig):
    def __init__(self):
        super().__init__()
        self.model_config_path = os.environ.get("STB200_EVAL_MODEL", "/models/Qwen3-8B")
        self.max_seq_len = 131072
        self.vllm_gpu_memory_utilization = 0.9
        self.vllm_tp, self.vllm_dp = 1, 8
        self.vllm_enable_chunked_prefill = True
        self.vllm_enable_prefix_caching = True
        self.max_cache_size = 256


class Qwen3_1p7BEvalVLLMDeployConfig(Qwen3EvalVLLMDeployConfig):
    def __init__(self):
        super().__init__()
        self.model_config_path = os.environ.get("STB200_EVAL_MODEL", "/models/Qwen3-1.7B")
        self.max_seq_len = 65536


class EvalTokenizerConfig(TokenizerConfig):
    tokenizer_path = Ref("...vllm_cfg.model_config_path")


class Qwen3SimpleBenchmarksEvalConfig(SimpleBenchmarksEvalConfig):
    tokenizer_cfg = EvalTokenizerConfig
    num_concurrent_requests = 4096


class Exp(BaseExp):
    vllm_cfg: VLLMDeployConfig = Qwen3EvalVLLMDeployConfig
    resource_cfg = EvalResourceConfig
    vllm_router_cfg: VLLMRouterConfig = VLLMRouterConfig
    eval_cfg = Qwen3SimpleBenchmarksEvalConfig
    log_dir = "./eval_logs/"

    def entrypoint(self) -> None:
        self.update_from_args()
        role = os.environ.get("ROLE", "evaluator")
        if role == "router":
            self.vllm_router_cfg.run()
        elif role == "vllm":
            self.vllm_cfg.run_as_worker()
        elif role == "evaluator":
            self.sanity_check()
            logger.info("waiting for the inference servers to register ...")
            self.vllm_cfg.build_cli().wait_for_server()
            logger.info(f"eval results: {self.eval_cfg.eval()}")
        else:
            raise ValueError(f"unknown ROLE: {role}")


class Exp1p7B(Exp):
    vllm_cfg = Qwen3_1p7BEvalVLLMDeployConfig


if __name__ == "__main__":
    Exp().entrypoint()
