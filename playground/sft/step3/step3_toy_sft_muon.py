"""The Step-3.5 toy model (48 layers at toy widths) SFT run with Muon on the hidden matrices: one 8-GPU node, TP=8 +
SP, EP=8, 8 sequences of 64k packed tokens per step, full recompute (reference
``playground/sft/step3/step3_toy_sft_step3_data_muon.py``)."""
from playground.data.sft.chat_sft_data import ChatSFTDataConfig
from playground.pretrain.step3p5.step3p5_toy import Step3p5ToyModelConfig
from playground.sft.qwen3.qwen3_sft_base import Exp as BaseExp
from playground.sft.step3.muon_optimizer import MuonGradientManagerConfig
from steptronoss_b200.exp.ntp import MoEPretrainMetricConfig


class Exp(BaseExp):
    model_cfg = Step3p5ToyModelConfig
    data_cfg = ChatSFTDataConfig
    optimizer_cfg = MuonGradientManagerConfig
    metric_cfg = MoEPretrainMetricConfig

    def __init__(self):
        super().__init__()
        t = self.trainer_cfg
        t.micro_batch_size = 1
        t.global_batch_size = 8
        t.global_seq_length = 65536
        t.train_iters = 1000
        t.log_interval = 1
        c = self.checkpoint_cfg
        c.load_option.none(but=["model"])
        c.save_safetensors = True
        c.save_dir = "./checkpoints/"
        c.save_option.all()
        c.save_interval = 100
        self.profiler_cfg.timing_log_level = 2
        self.model_cfg.recompute = True

    def configure_optimizable(self):
        from steptronoss_b200.utils.optimizable import set_optimization

        set_optimization(AttentionCore="flash-attn")       # the reference's switch here: the kernel path


if __name__ == "__main__":
    Exp().train()
