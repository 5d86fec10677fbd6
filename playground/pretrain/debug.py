"""A two-layer decoder on synthetic data that runs anywhere, CPU included: the quickest way to see the trainer,
the logger and the checkpointer work (reference ``playground/pretrain/debug.py``).

    python -m playground.pretrain.debug trainer_cfg.train_iters=20   # from the repository root
"""
import torch

from playground.pretrain.qwen3.qwen3_8b import Exp as Qwen3Exp


class Exp(Qwen3Exp):
    def __init__(self):
        super().__init__()
        m = self.model_cfg
        m.num_layers, m.hidden_size = 2, 256
        m.params_dtype = torch.bfloat16 if torch.cuda.is_available() else torch.float32
        m.parallel_cfg.tensor_model_parallel_size = 1
        m.tp_cfg.sequence_parallel = False
        a = m.attn_cfg
        a.num_attention_heads, a.num_attention_groups, a.head_dim, a.hidden_size = 2, 1, 128, 256
        m.ffn_cfg.hidden_size, m.ffn_cfg.ffn_hidden_size = 256, 512
        for e in (m.tok_embed_cfg, m.out_embed_cfg):
            e.vocab_size, e.hidden_size = 4096, 256
        t = self.trainer_cfg
        t.global_batch_size, t.global_seq_length, t.train_iters, t.log_interval = 4, 512, 10, 1
        t.writer_backend = []
        self.data_cfg.min_doc_len, self.data_cfg.max_doc_len = 32, 512
        self.scheduler_cfg.lr = 1e-3
        self.resource_cfg.gpu = 1


if __name__ == "__main__":
    Exp().train()
