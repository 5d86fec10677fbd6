"""Rotary tables: the YaRN rule that ``ntk_interp_ratio`` switches on, and the stand-alone rotary module."""
import math

import pytest
import torch

from steptronoss_b200.models.common.rope import (RoPEConfig, RotaryEmbedding, YARNRoPE, ntk_by_rotations_inv_freq,
                                                 ropen_linspace)


def test_half_open_linspace():
    assert torch.allclose(ropen_linspace(0, 1, 4), torch.tensor([0.0, 0.25, 0.5, 0.75]))


def test_ntk_rule_keeps_fast_channels_and_slows_the_rest():
    theta, dim, S, ratio = 10000.0, 64, 4096, 4.0
    inv = 1.0 / theta ** ropen_linspace(0, 1, dim // 2, dtype=torch.float64)
    out = ntk_by_rotations_inv_freq(inv, S, ratio, beta_fast=32, beta_slow=1)
    turns = S * inv / (2 * math.pi)
    assert torch.equal(out[turns >= 32], inv[turns >= 32])                         # many turns: untouched
    assert torch.allclose(out[turns <= 1], inv[turns <= 1] / ratio)                # less than one turn: interpolated
    mid = (turns > 1) & (turns < 32)
    assert mid.any() and ((out[mid] < inv[mid]) & (out[mid] > inv[mid] / ratio)).all()
    i = int(mid.nonzero()[0])
    w = (turns[i] - 1) / 31
    assert float(out[i]) == pytest.approx(float(inv[i] * w + inv[i] / ratio * (1 - w)), rel=1e-12)
    assert ntk_by_rotations_inv_freq(inv, S, 1.0) is inv
    # the attention module's tables follow the rule when the ratio is set, and are plain RoPE otherwise
    plain, scaled = RotaryEmbedding(dim, theta, S), RotaryEmbedding(dim, theta, S, ntk_interp_ratio=ratio)
    cp, _ = plain.tables(torch.device("cpu"), 16)
    cs, _ = scaled.tables(torch.device("cpu"), 16)
    assert torch.allclose(cp[:, 0], cs[:, 0]) and not torch.allclose(cp[:, -1], cs[:, -1])
    assert torch.allclose(cs[5], torch.cos(5 * out).float(), atol=1e-6)


def test_rotary_module_against_the_complex_rotation():
    torch.manual_seed(0)
    B, S, H, C, theta = 2, 12, 3, 16, 100.0
    x = torch.randn(B, S, H, C)
    rope = YARNRoPE(C, theta)
    out = rope(x)
    freq = 1.0 / theta ** ropen_linspace(0, 1, C // 2)
    ang = torch.outer(torch.arange(S).float(), freq)
    z = torch.complex(x[..., : C // 2], x[..., C // 2:]) * torch.polar(torch.ones_like(ang), ang)[None, :, None, :]
    assert torch.allclose(out, torch.cat([z.real, z.imag], -1), atol=1e-5)
    pos = torch.tensor([0, 1, 2, 3, 0, 1, 2, 0, 1, 2, 3, 4])                       # three packed documents
    packed = rope(x, position_id=pos)
    assert torch.allclose(packed[:, 4:7], rope(x[:, 4:7]), atol=1e-5)          # the second document restarts at 0
    adj = YARNRoPE(C, theta, use_adjacent_pair=True)(x)
    paired = x.view(B, S, H, C // 2, 2).transpose(4, 3).reshape(B, S, H, C)
    assert torch.allclose(adj, rope(paired), atol=1e-6)
    half = rope(x.to(torch.bfloat16))
    assert half.dtype == torch.bfloat16 and torch.allclose(half.float(), out, atol=0.05)
    cfg = RoPEConfig()
    cfg.dim, cfg.theta, cfg.ntk_interp_ratio, cfg.max_position_embeddings = C, theta, 2.0, 64
    built = cfg.build_model()
    assert isinstance(built, YARNRoPE) and not torch.allclose(built(x), out)
    with pytest.raises(ValueError):
        RotaryEmbedding(C, theta, 0, ntk_interp_ratio=2.0)
