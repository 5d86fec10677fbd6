"""Step-3.5 debug SFT that mirrors the flash model's one-node path: six layers at the flash model's widths (hidden
4096, 288 experts of 1280 + a shared expert, sliding window on four of the six), CP=8 without tensor parallelism, EP=8,
experts forced to a balanced load, 128k-token sequences, Adam, no checkpoints written
(reference ``playground/sft/step3/step3_toy_sft_step3_data.py``)."""
from playground.data.sft.chat_sft_data import ChatSFTDataConfig
from playground.pretrain.step3p5.step3p5_toy import Step3p5ToyModelConfig
from playground.sft.qwen3.qwen3_sft_base import Exp as BaseExp
from steptronoss_b200.exp.ntp import MoEPretrainMetricConfig


class Exp(BaseExp):
    model_cfg = Step3p5ToyModelConfig
    data_cfg = ChatSFTDataConfig
    metric_cfg = MoEPretrainMetricConfig

    def __init__(self):
        super().__init__()
        t = self.trainer_cfg
        t.micro_batch_size = 1
        t.global_batch_size = 32
        t.global_seq_length = 128 * 1024
        t.train_iters = None                  # one pass over the data
        t.log_interval = 1
        m = self.model_cfg
        m.num_layers = 6
        m.hidden_size = 4096
        m.swa_layer_list = [False, True, True, True, False, True]
        m.attn_cfg.num_attention_heads = 64
        m.attn_cfg.num_attention_groups = 8
        m.attn_cfg.head_dim = 128
        m.swa_cfg.num_attention_heads = 96
        m.ffn_cfg.ffn_hidden_size = 11264
        m.moe_cfg.moe_num_experts = 288
        m.moe_cfg.moe_hidden_size = 1280
        m.moe_cfg.share_expert_dim = 1280
        m.moe_cfg.moe_layer_list = list(range(6))
        m.moe_cfg.force_balance = True
        m.recompute = True
        m.parallel_cfg.context_parallel_size = 8
        m.parallel_cfg.tensor_model_parallel_size = 1
        m.tp_cfg.sequence_parallel = False
        c = self.checkpoint_cfg
        c.load_option.none(but=["model"])
        c.save_safetensors = False
        c.save_dir = "./checkpoints/"
        c.save_option.none()
        c.save_interval = 100
        c.auto_resume = False
        self.profiler_cfg.timing_log_level = 2

    def configure_optimizable(self):
        from steptronoss_b200.utils.optimizable import set_optimization

        # the reference's switches for this experiment; here they all name the kernel paths and the peer dispatcher
        set_optimization(routed_grouped_ffn="fused", moe_weighted_gather="triton", TokenDispatcher="deep_ep",
                         grouped_gemm="nv_grouped_gemm", AttentionCore="flash-attn-3")


if __name__ == "__main__":
    Exp().train()
