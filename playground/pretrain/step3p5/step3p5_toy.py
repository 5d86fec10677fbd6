"""Step-3.5 at toy size with every feature of the flash model: 48 layers of hidden 2048 (sliding window on three
layers of every four), 32 / 48 query heads, 128 experts of width 768 + a shared expert on layers 1..47 with a live
aux-loss-free router bias, dense SwiGLU 7168 on layer 0.  Layout for one 8-GPU node: TP=8 with sequence
parallelism, EP=8."""
from playground.pretrain.step3p5.step3p5_flash import Step3p5FlashModelConfig


class Step3p5ToyModelConfig(Step3p5FlashModelConfig):
    def __init__(self):
        super().__init__()
        self.hidden_size = 2048
        self.num_layers = 48
        self.swa_layer_list = [True, True, True, False] * 12
        self.attn_cfg.num_attention_heads = 32
        self.swa_cfg.num_attention_heads = 48
        m = self.moe_cfg
        m.moe_num_experts = 128
        m.moe_hidden_size = 768
        m.share_expert_dim = 768
        m.moe_layer_list = list(range(1, 48))
        m.router_bias_update_rate = 0.1
        m.expert_swiglu_limits = {}
        m.shared_expert_swiglu_limit = {}
        self.ffn_cfg.ffn_hidden_size = 7168
        p = self.parallel_cfg
        p.tensor_model_parallel_size = 8
        p.pipeline_model_parallel_size = 1
        p.virtual_pipeline_model_parallel_size = 1
        p.context_parallel_size = 1
        p.expert_model_parallel_size = 8
        p.expert_tensor_parallel_size = 1
        self.tp_cfg.sequence_parallel = True
