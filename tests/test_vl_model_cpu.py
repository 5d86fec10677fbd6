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


def test_hf_weights_of_text_vision_and_projector_round_trip():
    """Export in HF spelling (``model.*`` / ``lm_head``, ``vision_model.*`` with fused ``in_proj``,
    ``vit_large_projector``), load into a differently initialised model: every parameter comes back."""
    from steptronoss_b200.models.qwen_vl import QwenImageInsertModelConfig
    from steptronoss_b200.parallel.state import PM

    PM.initialize()
    src_cfg = _cfg()
    cfg = QwenImageInsertModelConfig()
    cfg.merge(src_cfg.to_dict())
    PM.set_mesh(cfg.parallel_cfg)
    a, b = cfg.build_model(), cfg.build_model()
    a.init_weights(1, 0.02)
    b.init_weights(2, 0.02)
    with torch.no_grad():                                   # the encoder keeps torch's own initialisation: make the two differ
        for p in b.encoder.parameters():
            p.add_(0.5)
        b.tok_embeddings.align_projector.weight.add_(0.5)
    hf = a.hf_state_dict()
    assert "vit_large_projector.weight" in hf and "model.embed_tokens.weight" in hf
    assert "vision_model.transformer.resblocks.0.attn.in_proj_weight" in hf
    assert "vision_model.transformer.resblocks.0.mlp.c_fc.weight" in hf and "vision_model.conv1.weight" in hf
    assert not any(k.startswith("encoder.") or "qkv_proj" in k for k in hf)
    skipped = b.load_hf_state_dict({k: v.clone() for k, v in hf.items()})
    assert skipped == []
    pa, pb = dict(a.named_parameters()), dict(b.named_parameters())
    assert set(pa) == set(pb)
    for k in pa:
        assert torch.equal(pa[k], pb[k]), k


def test_step3v_exports_vision_rules_in_front_of_the_step3p5_mapping():
    from steptronoss_b200.models.step3v import Step3VModelConfig
    from steptronoss_b200.parallel.state import PM
    from tests.test_step3p5_cpu import _make

    PM.initialize()
    text = _make().model_cfg
    cfg = Step3VModelConfig()
    d = text.to_dict()
    d.pop("tok_embed_cfg", None)
    cfg.merge(d)
    t = cfg.tok_embed_cfg
    t.vocab_size, t.hidden_size, t.img_start_token = 256, 64, 3
    e = t.encoder_cfg
    e.image_size, e.patch_size, e.hidden_size, e.ffn_hidden_size, e.num_layers, e.num_attention_heads = 32, 4, 16, 32, 1, 2
    e.vit_downsampler_hidden_dim, e.output_dim = 24, 20
    PM.set_mesh(cfg.parallel_cfg)
    a, b = cfg.build_model(), cfg.build_model()
    a.init_weights(1, 0.02)
    b.init_weights(2, 0.02)
    hf = a.hf_state_dict()
    assert "vit_large_projector.weight" in hf and any(k.startswith("vision_model.") for k in hf)
    assert any(k.startswith("model.layers.1.") for k in hf)
    b.load_hf_state_dict({k: v.clone() for k, v in hf.items()})
    pa, pb = dict(a.named_parameters()), dict(b.named_parameters())
    differ = [k for k in pa if not torch.equal(pa[k], pb[k])]
    assert all("router_bias" in k or "expert_bias" in k for k in differ), differ
