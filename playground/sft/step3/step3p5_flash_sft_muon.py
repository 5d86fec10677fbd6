"""Step-3.5-Flash SFT with Muon on 128k-token sequences: 45 layers over PP=8 x VPP=3 (layers per virtual stage given
explicitly, the last stage kept light because it also holds the head and the loss), TP=8 with sequence parallelism,
EP=8, no context parallelism, cosine schedule (reference ``playground/sft/step3/step3p5_flash_sft_step3_data_muon.py``).
A 64-GPU job: ``resource_cfg.replica = 8``."""
from playground.data.sft.chat_sft_data import ChatSFTDataConfig
from playground.pretrain.step3p5.step3p5_flash import Step3p5FlashModelConfig
from playground.sft.qwen3.qwen3_sft_base import Exp as BaseExp
from playground.sft.step3.muon_optimizer import MuonGradientManagerConfig
from steptronoss_b200.exp.lr_schedulers import CosineSchedulerConfig
from steptronoss_b200.exp.ntp import MoEPretrainMetricConfig


class Step3p5FlashSFTModelConfig(Step3p5FlashModelConfig):
    layers_per_virtual_stage: list = [2] * 22 + [1, 0]
    """45 layers over PP=8 x VPP=3 = 24 virtual stages: two per slot, one on stage 6's last chunk and none on stage
    7's, which moves memory off the last pipeline stage"""

    def __init__(self):
        super().__init__()
        self.parallel_cfg.context_parallel_size = 1
        self.parallel_cfg.tensor_model_parallel_size = 8
        self.tp_cfg.sequence_parallel = True

    def pp_vp_allocation(self, abs_pp_rank: int) -> list:
        if len(self.layers_per_virtual_stage) != 24 or sum(self.layers_per_virtual_stage) != self.num_layers:
            raise ValueError("layers_per_virtual_stage must name 24 virtual stages holding every layer once")
        return [{} for _ in range(self.layers_per_virtual_stage[abs_pp_rank])]


class Exp(BaseExp):
    model_cfg = Step3p5FlashSFTModelConfig
    data_cfg = ChatSFTDataConfig
    optimizer_cfg = MuonGradientManagerConfig
    scheduler_cfg = CosineSchedulerConfig
    metric_cfg = MoEPretrainMetricConfig

    def __init__(self):
        super().__init__()
        self.resource_cfg.replica = 8
        self.resource_cfg.envs = {**(self.resource_cfg.envs or {}), "PYTORCH_CUDA_ALLOC_CONF": "expandable_segments:True",
                                  "CUDA_DEVICE_MAX_CONNECTIONS": "1"}
        t = self.trainer_cfg
        t.micro_batch_size = 1
        t.global_batch_size = 32
        t.global_seq_length = 128 * 1024
        t.train_iters = None                 # one pass over the data
        t.log_interval = 1
        self.model_cfg.recompute = True
        s = self.scheduler_cfg
        s.lr = 1e-5
        s.min_lr = 5e-6
        s.weight_decay = 0.1
        s.warmup_schedule = 140
        s.scheduler_unit = "iter"
        s.total_schedule = None
        c = self.checkpoint_cfg
        c.load_option.none(but=["model"])
        c.save_safetensors = True
        c.save_dir = "./checkpoints/"
        c.save_option.all()
        c.save_interval = 500


if __name__ == "__main__":
    Exp().train()
