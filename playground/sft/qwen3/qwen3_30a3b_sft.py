"""Qwen3-30B-A3B SFT on chat data: EP=8, attention data parallel, 8 sequences of 64k packed tokens per step as in the
reference's experiment (``playground/sft/qwen3/qwen3_30a3b_sft_step3_data.py``).  Its full recompute is replaced by
recomputing the two norms per layer: 180 GB hold the other activations of a 64k sequence."""
from playground.data.sft.chat_sft_data import ChatSFTDataConfig
from playground.pretrain.qwen3.qwen3_30a3b import Qwen3_30A3BConfig
from playground.sft.qwen3.qwen3_sft_base import Exp as BaseExp
from steptronoss_b200.exp.ntp import MoEPretrainMetricConfig


class Exp(BaseExp):
    model_cfg = Qwen3_30A3BConfig
    data_cfg = ChatSFTDataConfig
    metric_cfg = MoEPretrainMetricConfig

    def __init__(self):
        super().__init__()
        t = self.trainer_cfg
        t.log_interval = 1
        t.micro_batch_size = 1
        t.global_batch_size = 8
        t.global_seq_length = 65536
        self.model_cfg.moe_cfg.dispatcher = "peer"
        self.model_cfg.recompute = ["attn_norm", "ffn_norm"]
        s = self.scheduler_cfg
        s.lr = 1e-5
        s.min_lr = 1e-6
        s.warmup_schedule = 100
        c = self.checkpoint_cfg
        c.load_option.none(but=["model"])
        c.save_safetensors = True
        c.save_dir = "./checkpoints/"
        c.save_option.all()
        c.save_interval = 100


if __name__ == "__main__":
    Exp().train()
