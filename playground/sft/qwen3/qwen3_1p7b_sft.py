"""Qwen3-1.7B SFT on chat data, sequences packed to 128k tokens under TP=8 (reference
``playground/sft/qwen3/qwen3_1p7b_sft_step3_data.py``).  Start from HF weights with
``checkpoint_cfg.load_safetensors=/path/to/Qwen3-1.7B-Base``.

    torchrun --nproc-per-node 8 -m playground.sft.qwen3.qwen3_1p7b_sft checkpoint_cfg.load_safetensors=/models/Qwen3-1.7B-Base
"""
from playground.data.sft.chat_sft_data import ChatSFTDataConfig
from playground.pretrain.qwen3.qwen3_1p7b import Qwen3_1p7BConfig
from playground.sft.qwen3.qwen3_sft_base import Exp as BaseExp


class Exp(BaseExp):
    model_cfg = Qwen3_1p7BConfig
    data_cfg = ChatSFTDataConfig

    def __init__(self):
        super().__init__()
        t = self.trainer_cfg
        t.log_interval = 1
        t.micro_batch_size = 1
        t.global_batch_size = 32
        t.global_seq_length = 128 * 1024
        self.model_cfg.parallel_cfg.tensor_model_parallel_size = 8
        s = self.scheduler_cfg
        s.lr = 1e-5
        s.min_lr = 1e-6
        s.warmup_schedule = 100
        c = self.checkpoint_cfg
        c.load_option.none(but=["model"])
        c.save_safetensors = True
        c.save_dir = "./checkpoints/"
        c.save_option.all()
        c.save_interval = 1000


if __name__ == "__main__":
    Exp().train()
