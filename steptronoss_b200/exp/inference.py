"""Deployment configuration of the inference replicas that generate rollouts and evaluation answers.

Reference: ``steptronoss/exp/inference.py:8-190``.  The replicas are vLLM OpenAI-compatible servers started
by :class:`steptronoss_b200.generation.vllm.vllm_controller.VLLMController`, registered with the
experiment's router and addressed through it by :class:`~steptronoss_b200.generation.vllm.vllm_client.VLLMClient`.
Training weights reach them as a safetensors dump in ``hot_path`` followed by a ``reload_weights`` RPC.
"""
from __future__ import annotations

import json

import torch

from ..config import Config, Ref
from ..utils.logger import logger


class BaseInferenceConfig(Config):
    max_seq_len: int = 65536
    """prefill + decode length limit of the engine"""
    max_decode_steps: int | None = None
    """generated-token limit; ``None`` = ``max_seq_len - prompt_len``"""
    max_cache_size: int = 64
    """decode batch size (``max_num_seqs``)"""
    shuffle_all_samples: bool = True
    temperature: float = 1.0


class VLLMDeployConfig(BaseInferenceConfig):
    router_addr_key: str = "default"
    """key under which the router publishes ``host:port`` in the experiment store"""
    model_config_path: str = ""
    load_weight_from_config_path: bool = True
    tokenizer_path = Ref(".model_config_path")
    vllm_tp: int = 8
    vllm_pp: int = 1
    vllm_dp: int = 1
    enable_expert_parallel: bool = False
    vllm_gpu_memory_utilization: float = 0.95
    vllm_enable_chunked_prefill: bool = True
    vllm_max_num_batched_tokens: int = 8192
    vllm_enable_prefix_caching: bool = True
    vllm_enforce_eager: bool = False
    vllm_trust_remote_code: bool = True
    enable_auto_tool_choice: bool = False
    toolcall_parser: str | None = None
    quantize: str | None = None
    block_size: int | None = None
    enable_log_requests: bool = False
    enable_reasoning: bool = False
    reasoning_parser: str | None = None
    model_name_template: str = "deployed-model-{EXP_ID}"
    hot_path: str | None = None
    vllm_hf_overrides: dict = {}
    vllm_mtp_num_tokens: int = 0
    vllm_mtp_method: str = ""

    def sanity_check(self):
        super().sanity_check()
        if torch.cuda.is_available():
            gpus = torch.cuda.device_count()
            if self.vllm_dp * self.vllm_tp != gpus:
                logger.warning(f"Using DP={self.vllm_dp} & TP={self.vllm_tp} for vLLM, but detected {gpus} GPU on node!")
        if self.enable_auto_tool_choice:
            assert self.toolcall_parser

    def run_as_worker(self):
        """Deploy one server on this node and register it with the experiment's router (blocks)."""
        from ..generation.vllm.vllm_controller import VLLMController

        VLLMController(cfg=self).start()

    @property
    def model_name(self) -> str:
        from ..utils.comm_utils import get_exp_id

        return self.model_name_template.format(EXP_ID=get_exp_id())

    def build_cli(self):
        from ..generation.vllm.vllm_client import VLLMClient

        return VLLMClient(cfg=self)

    def get_entrypoint_command_and_envs(self) -> tuple[str, dict]:
        envs: dict = {}
        cmd = [
            "vllm serve", f"{self.model_config_path}", "--port $PORT_SERVING",
            f"--served-model-name {self.model_name}", f"--max-model-len {self.max_seq_len}",
            f"--tensor-parallel-size {self.vllm_tp}", f"--gpu-memory-utilization {self.vllm_gpu_memory_utilization}",
            f"--max-num-seqs {self.max_cache_size}", f"--data-parallel-size {self.vllm_dp}",
            f"--max-num-batched-tokens {self.vllm_max_num_batched_tokens}",
            "--disable-cascade-attn", "--disable-uvicorn-access-log",
        ]
        if self.vllm_pp > 1:
            cmd.append(f"--pipeline-parallel-size {self.vllm_pp}")
        if self.vllm_hf_overrides:
            envs["HF_OVERRIDES"] = f"'{json.dumps(self.vllm_hf_overrides)}'"
            cmd.append("--hf-overrides $HF_OVERRIDES")
        if self.tokenizer_path:
            cmd.append(f"--tokenizer {self.tokenizer_path}")
        if self.vllm_trust_remote_code:
            cmd.append("--trust-remote-code")
        if self.toolcall_parser:
            cmd += ["--enable-auto-tool-choice", f"--tool-call-parser {self.toolcall_parser}"]
        if self.reasoning_parser:
            cmd.append(f"--reasoning-parser {self.reasoning_parser}")
        if not self.load_weight_from_config_path:
            cmd.append("--load-format dummy")
        if self.vllm_enable_chunked_prefill:
            cmd.append("--enable-chunked-prefill")
        if self.vllm_enforce_eager:
            cmd.append("--enforce-eager")
        if not self.vllm_enable_prefix_caching:
            cmd.append("--no-enable-prefix-caching")
        if self.quantize:
            cmd.append(f"--quantization {self.quantize}")
        if self.block_size:
            cmd.append(f"--block-size {self.block_size}")
        if self.enable_log_requests:
            cmd.append("--enable-log-requests")
        if self.enable_expert_parallel:
            cmd.append("--enable-expert-parallel")
        if self.vllm_mtp_num_tokens > 0:
            spec = json.dumps({"num_speculative_tokens": self.vllm_mtp_num_tokens, "method": self.vllm_mtp_method})
            envs["SPECULATIVE_CONFIG"] = f"'{spec}'"
            cmd.append("--speculative-config $SPECULATIVE_CONFIG")
        return " ".join(cmd), envs

    def deploy_training_model(self, models) -> None:
        """Dump the training weights as safetensors into ``hot_path`` (collective) and have every replica
        reload them."""
        from ..checkpointing.hf_checkpoint import dump_safetensors
        from ..parallel.state import PM

        cli = self.build_cli()
        dump_safetensors(models, self.hot_path, config_source=self.model_config_path or None)
        if PM.world_rank == 0:
            cli.wait_for_server()
            cli.reload_weights(self.hot_path)
        cli.wait_for_server()
