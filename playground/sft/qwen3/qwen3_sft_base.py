"""Base of the Qwen3 SFT experiments (reference ``playground/sft/qwen3/qwen3_sft_base.py``): one 8-GPU node,
next-token trainer, ZeRO-1 Adam, constant schedule with warm-up; subclasses set ``model_cfg`` / ``data_cfg`` and
the checkpoint to start from."""
from steptronoss_b200.exp.base_exp import GradientManagerConfig, ProfilerConfig
from steptronoss_b200.exp.checkpointing import CheckpointConfig
from steptronoss_b200.exp.lr_schedulers import ConstantSchedulerConfig
from steptronoss_b200.exp.ntp import NTPTrainerConfig, PretrainMetricConfig
from steptronoss_b200.exp.resources import TorchrunResourceConfig
from steptronoss_b200.exp.sft import SFTExp


class OneNodeResourceConfig(TorchrunResourceConfig):
    def __init__(self):
        super().__init__()
        self.replica = 1
        self.gpu = 8


class Exp(SFTExp):
    log_dir = "./tensorboard_logs/"
    resource_cfg = OneNodeResourceConfig
    trainer_cfg = NTPTrainerConfig
    optimizer_cfg = GradientManagerConfig
    scheduler_cfg = ConstantSchedulerConfig
    checkpoint_cfg = CheckpointConfig
    metric_cfg = PretrainMetricConfig
    profiler_cfg = ProfilerConfig


if __name__ == "__main__":
    Exp().train()
