"""Step-3.5-Flash SFT with Muon: 45 layers over PP=8 x VPP=3 (layers per virtual stage given explicitly), CP=8,
EP=8, 128k-token sequences (reference ``playground/sft/step3/step3p5_flash_sft_step3_data_muon.py``).  A 64-GPU job:
``resource_cfg.replica = 8``."""
from playground.data.sft.chat_sft_data import ChatSFTDataConfig
from playground.pretrain.step3p5.step3p5_flash import Step3p5FlashModelConfig
from playground.sft.qwen3.qwen3_sft_base import Exp as BaseExp
from playground.sft.step3.muon_optimizer import MuonGradientManagerConfig
from steptronoss_b200.exp.ntp import MoEPretrainMetricConfig


class Step3p5FlashSFTModelConfig(Step3p5FlashModelConfig):
    layers_per_virtual_stage: list = [2] * 21 + [1] * 3
    """45 layers over PP=8 x VPP=3 = 24 virtual stages"""

    def pp_vp_allocation(self, abs_pp_rank: int) -> list:
        return [{} for _ in range(self.layers_per_virtual_stage[abs_pp_rank])]


class Exp(BaseExp):
    model_cfg = Step3p5FlashSFTModelConfig
    data_cfg = ChatSFTDataConfig
    optimizer_cfg = MuonGradientManagerConfig
    metric_cfg = MoEPretrainMetricConfig

    def __init__(self):
        super().__init__()
        self.resource_cfg.replica = 8
        t = self.trainer_cfg
        t.micro_batch_size = 1
        t.global_batch_size = 64
        t.global_seq_length = 128 * 1024
        t.train_iters = 1000
        t.log_interval = 1
        self.model_cfg.recompute = True
        s = self.scheduler_cfg
        s.lr = 2e-5
        s.min_lr = 2e-6
        s.weight_decay = 0.1
        s.warmup_schedule = 50
        c = self.checkpoint_cfg
        c.load_option.none(but=["model"])
        c.save_safetensors = True
        c.save_dir = "./checkpoints/"
        c.save_option.all()
        c.save_interval = 100


if __name__ == "__main__":
    Exp().train()
