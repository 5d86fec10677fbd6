"""2-D rotary embedding of the vision encoder and its effect on the attention block."""
import torch


def test_rope2d_is_a_rotation_that_depends_on_relative_grid_offsets():
    from steptronoss_b200.models.common.vit import EncoderRope2D

    torch.manual_seed(0)
    rope = EncoderRope2D(dim=8, max_grid_height=4, max_grid_width=4)
    q, k = torch.randn(1, 4, 2, 8), torch.randn(1, 4, 2, 8)                    # [B, L, heads, D], a 2x2 grid
    qo, ko = rope(q, k, grid_hw=(2, 2))
    assert qo.shape == q.shape and torch.isfinite(qo).all()
    assert torch.allclose(qo[:, 0], q[:, 0]) and torch.allclose(ko[:, 0], k[:, 0])  # grid origin: angle zero
    assert not torch.allclose(qo[:, 1:], q[:, 1:])
    assert torch.allclose(qo.norm(dim=-1), q.norm(dim=-1), atol=1e-5)               # pairs are rotated, not scaled
    # a 2x2 window uses the rows 0, 1, 4, 5 of the 4x4 table
    assert torch.equal(rope.freqs((2, 2), "cpu"), rope.freqs_cache[[0, 1, 4, 5]])
    # the score of one (query, key) pair depends on their offset only: place the same vectors one column further right
    full = EncoderRope2D(dim=8, max_grid_height=4, max_grid_width=4)
    a, b = torch.randn(8), torch.randn(8)

    def score(pos_q, pos_k):
        qq, kk = torch.zeros(1, 16, 1, 8), torch.zeros(1, 16, 1, 8)
        qq[0, pos_q, 0], kk[0, pos_k, 0] = a, b
        rq, rk = full(qq, kk, grid_hw=(4, 4))
        return float((rq[0, pos_q, 0] * rk[0, pos_k, 0]).sum())

    assert abs(score(0, 5) - score(1, 6)) < 1e-5 and abs(score(0, 5) - score(10, 15)) < 1e-5   # offset (+1 row, +1 col)
    assert abs(score(0, 5) - score(0, 6)) > 1e-4


def test_rope2d_leaves_the_class_token_alone():
    from steptronoss_b200.models.common.vit import EncoderRope2D

    rope = EncoderRope2D(dim=8, max_grid_height=2, max_grid_width=2, use_cls_token=True)
    q = torch.randn(1, 5, 1, 8)
    qo, _ = rope(q, q.clone(), grid_hw=(2, 2))
    assert torch.equal(qo[:, 0], q[:, 0]) and not torch.allclose(qo[:, 1], q[:, 1])   # with a class token the grid starts at 1


def test_attention_block_with_and_without_rope():
    from steptronoss_b200.models.common.vit import VisionAttention, VisionTransformerConfig
    from steptronoss_b200.parallel.state import PM

    PM.initialize()
    cfg_plain, cfg_rope = VisionTransformerConfig(), VisionTransformerConfig()
    for c, on in ((cfg_plain, False), (cfg_rope, True)):
        c.image_size, c.patch_size, c.hidden_size, c.num_attention_heads, c.use_cls_token, c.use_rope2d = 4, 2, 8, 2, False, on
    PM.set_mesh(cfg_plain.parallel_cfg)
    torch.manual_seed(3)
    plain, rope = VisionAttention(cfg_plain), VisionAttention(cfg_rope)
    for p in plain.parameters():
        torch.nn.init.normal_(p, std=0.5)
    rope.load_state_dict(plain.state_dict(), strict=True)                         # the rope holds no parameters
    x = torch.randn(1, 4, 8)
    a, b = plain(x, grid_hw=(2, 2)), rope(x, grid_hw=(2, 2))
    assert a.shape == b.shape == (1, 4, 8) and torch.isfinite(b).all() and not torch.allclose(a, b)


def test_attention_dropout_acts_in_training_only():
    from steptronoss_b200.models.common.vit import VisionAttention, VisionTransformerConfig
    from steptronoss_b200.parallel.state import PM

    PM.initialize()
    cfg = VisionTransformerConfig()
    cfg.image_size, cfg.patch_size, cfg.hidden_size, cfg.num_attention_heads, cfg.use_cls_token = 4, 2, 8, 2, False
    cfg.attention_dropout = 0.5
    PM.set_mesh(cfg.parallel_cfg)
    torch.manual_seed(0)
    attn = VisionAttention(cfg)
    for p in attn.parameters():
        torch.nn.init.normal_(p, std=0.5)
    x = torch.randn(2, 4, 8)
    attn.eval()
    a, b = attn(x, (2, 2)), attn(x, (2, 2))
    assert torch.equal(a, b)                                       # evaluation: no dropout
    attn.train()
    c, d = attn(x, (2, 2)), attn(x, (2, 2))
    assert not torch.allclose(c, d) and not torch.allclose(c, a)   # training: a fresh mask every call
    cfg.attention_dropout = 0.0
    plain = VisionAttention(cfg)
    plain.load_state_dict(attn.state_dict())
    plain.train()
    assert torch.allclose(plain(x, (2, 2)), a, atol=1e-5)          # both paths compute the same attention


def test_apply_rotary_emb_rotates_a_channel_range():
    from steptronoss_b200.models.common.vit import apply_rotary_emb, rotate_half

    x = torch.tensor([[1.0, 2.0, 3.0, 4.0, 5.0, 6.0]])
    assert rotate_half(x[:, :4]).tolist() == [[-2.0, 1.0, -4.0, 3.0]]
    quarter = torch.full((1, 2), torch.pi / 2)
    out = apply_rotary_emb(quarter, x, start_index=2)
    assert torch.allclose(out, torch.tensor([[1.0, 2.0, -4.0, 3.0, 5.0, 6.0]]), atol=1e-6)     # 90 degrees on channels 2..3
    assert torch.allclose(apply_rotary_emb(quarter, x, start_index=2, scale=2.0)[:, 2:4], torch.tensor([[-8.0, 6.0]]), atol=1e-5)
    half = apply_rotary_emb(quarter, x.to(torch.bfloat16))
    assert half.dtype == torch.bfloat16 and half[0, :2].tolist() == [-2.0, 1.0]
    import pytest

    with pytest.raises(ValueError):
        apply_rotary_emb(torch.zeros(1, 8), x)
