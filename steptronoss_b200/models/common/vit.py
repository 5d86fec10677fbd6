"""Vision transformer encoder for the vision-language models (reference ``steptronoss/model/common/vit.py``).

Patch embedding (a strided convolution = one GEMM over unfolded patches), optional CLS token, learned
positional embedding (bicubically resized to other grids), pre-norm blocks of full (non-causal) attention with
optional 2-D RoPE and a quick-GELU MLP, optional layer scale, then two strided convolutions that reduce the
patch grid 4x per side for the language projector.  Module and parameter names follow the reference so that
its checkpoints and HF mapping apply unchanged.

The projections run through ``ops.linear`` (the tcgen05 GEMM on GPU) and the attention through
``ops.attention`` with every image as one segment; head sizes other than 128 use the PyTorch restatement of
the attention (the hand-written kernel is specialised for 128).
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from ...config import Config
from ...exp.base_exp import ParallelConfig
from ...ops import linear
from ...ops.attention import attention, attention_reference
from ...parallel import mappings
from ...parallel.layers import set_tensor_model_parallel_attributes
from ...parallel.state import PM


def quick_gelu(x: torch.Tensor) -> torch.Tensor:
    return x * torch.sigmoid(1.702 * x)


def _rotate_pairs(x: torch.Tensor) -> torch.Tensor:
    x1, x2 = x[..., 0::2], x[..., 1::2]
    return torch.stack((-x2, x1), dim=-1).flatten(-2)


rotate_half = _rotate_pairs          # the reference's name: adjacent pairs (x0, x1) -> (-x1, x0)


def apply_rotary_emb(freqs: torch.Tensor, tensor: torch.Tensor, *, start_index: int = 0, scale: float = 1.0) -> torch.Tensor:
    """Rotate the channels ``[start_index, start_index + freqs.shape[-1])`` of a q / k tensor by the angles ``freqs``
    (adjacent-pair convention, fp32 arithmetic, result in the tensor's dtype); the channels left and right of the
    range pass through.  ``freqs`` broadcasts against the tensor (reference: model/common/vit.py:32-53)."""
    width = freqs.shape[-1]
    if start_index + width > tensor.shape[-1]:
        raise ValueError(f"feature dimension {tensor.shape[-1]} is too small for rot_dim {width} at {start_index}")
    ang = freqs.to(device=tensor.device, dtype=torch.float32)
    mid = tensor[..., start_index:start_index + width].float()
    mid = (mid * ang.cos() + _rotate_pairs(mid) * ang.sin()) * scale
    return torch.cat((tensor[..., :start_index], mid.to(tensor.dtype), tensor[..., start_index + width:]), dim=-1)


class EncoderRope2D(nn.Module):
    """Rotary embedding over a 2-D patch grid: half of the head dimension rotates with the column index, half
    with the row index (adjacent-pair convention); the CLS token, if any, is not rotated."""

    def __init__(self, dim: int, max_grid_height: int, max_grid_width: int, *, use_cls_token: bool = False,
                 theta: float = 10000, theta_rescale_factor: float = 1.0):
        super().__init__()
        self.dim, self.gh, self.gw, self.use_cls_token = dim, max_grid_height, max_grid_width, use_cls_token
        self.theta = theta * theta_rescale_factor ** (dim / (dim - 2))
        self.register_buffer("freqs_cache", self._table(), persistent=False)

    def _table(self) -> torch.Tensor:
        half = self.dim // 2
        inv = 1.0 / (self.theta ** (torch.arange(0, half, 2)[: half // 2].float() / half))
        off = 1.0 if self.use_cls_token else 0.0
        fh = ((torch.arange(self.gh).float() + off)[:, None] * inv).repeat_interleave(2, dim=-1)
        fw = ((torch.arange(self.gw).float() + off)[:, None] * inv).repeat_interleave(2, dim=-1)
        table = torch.cat([fw[None, :, :].expand(self.gh, self.gw, -1), fh[:, None, :].expand(self.gh, self.gw, -1)],
                          dim=-1).reshape(self.gh * self.gw, -1)
        if self.use_cls_token:
            table = torch.cat([torch.zeros(1, table.shape[-1]), table], dim=0)
        return table  # [tokens, dim]

    def freqs(self, grid_hw: tuple[int, int], device) -> torch.Tensor:
        if grid_hw == (self.gh, self.gw):
            return self.freqs_cache.to(device)
        rows = torch.arange(grid_hw[0], device=device).view(-1, 1)
        cols = torch.arange(grid_hw[1], device=device).view(1, -1)
        pos = (rows * self.gw + cols).reshape(-1)
        if self.use_cls_token:
            pos = torch.cat([torch.zeros(1, device=device, dtype=torch.long), pos + 1])
        return self.freqs_cache.to(device).index_select(0, pos)

    def forward(self, q: torch.Tensor, k: torch.Tensor, grid_hw: tuple[int, int]):
        """q, k ``[B, L, h, D]``."""
        f = self.freqs(grid_hw, q.device)[None, :, None, :]
        cos, sin = f.cos(), f.sin()

        def rot(t):
            tf = t.float()
            return (tf * cos + _rotate_pairs(tf) * sin).to(t.dtype)

        return rot(q), rot(k)


def interpolate_positional_embedding(pe: torch.Tensor, target_tokens: int, *, use_cls_token: bool) -> torch.Tensor:
    """``[tokens, C]`` or ``[1, tokens, C]`` on a square grid -> ``[1, target_tokens, C]`` (bicubic)."""
    if pe.dim() == 2:
        pe = pe.unsqueeze(0)
    if pe.shape[1] == target_tokens:
        return pe
    cls, grid = (pe[:, :1], pe[:, 1:]) if use_cls_token else (None, pe)
    src, dst = math.isqrt(grid.shape[1]), math.isqrt(target_tokens - (1 if use_cls_token else 0))
    if src * src != grid.shape[1]:
        raise ValueError(f"Expected square positional grid, got {grid.shape[1]} tokens")
    if dst * dst != target_tokens - (1 if use_cls_token else 0):
        raise ValueError(f"Expected square target grid, got {target_tokens} tokens")
    g = grid.reshape(1, src, src, -1).permute(0, 3, 1, 2).float()
    g = F.interpolate(g, size=(dst, dst), mode="bicubic", align_corners=False).to(pe.dtype)
    g = g.permute(0, 2, 3, 1).reshape(1, dst * dst, -1)
    return torch.cat([cls, g], dim=1) if cls is not None else g


class VisionTransformerParallelConfig(ParallelConfig):
    """The encoder's own mesh; by default every rank runs it un-sharded."""

    def __init__(self):
        super().__init__()
        self.tensor_model_parallel_size = 1
        self.pipeline_model_parallel_size = 1
        self.virtual_pipeline_model_parallel_size = 1
        self.context_parallel_size = 1
        self.expert_model_parallel_size = 1
        self.expert_tensor_parallel_size = 1


class VisionTransformerConfig(Config):
    parallel_cfg = VisionTransformerParallelConfig
    in_channels: int = 3
    image_size: int = 224
    patch_size: int = 14
    hidden_size: int = 1024
    ffn_hidden_size: int = 4096
    num_layers: int = 24
    num_attention_heads: int = 16
    vit_downsampler_hidden_dim: int = 2048
    output_dim: int = 4096
    layernorm_epsilon: float = 1e-5
    attention_dropout: float = 0.0
    use_rope2d: bool = False
    rope_theta: float = 10000
    rope_max_freq: int = 10
    rope_num_freqs: int = 1
    rope_theta_rescale_factor: float = 1.0
    layer_scale_init_value: float | None = None
    use_cls_token: bool = True
    use_ln_pre: bool = False
    patch_embed_bias: bool = True
    vit_downsampler1_kernel_size: int = 2
    vit_downsampler1_padding: int = 0
    vit_downsampler2_kernel_size: int = 3
    vit_downsampler2_padding: int = 1

    def build_model(self) -> "VisionTransformer":
        return VisionTransformer(cfg=self)


class LayerScale(nn.Module):
    def __init__(self, dim: int, init_value: float):
        super().__init__()
        self.gamma = nn.Parameter(torch.full((dim,), float(init_value)))

    def forward(self, x):
        return x * self.gamma


def _proj(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None) -> torch.Tensor:
    """``x @ weight.T (+ bias)`` over the last dimension."""
    if x.is_cuda and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16:
        y = linear(x.reshape(-1, x.shape[-1]), weight).view(*x.shape[:-1], weight.shape[0])
    else:
        y = F.linear(x, weight.to(x.dtype))
    return y if bias is None else y + bias.to(y.dtype)


class TPColumnLinear(nn.Module):
    def __init__(self, input_size: int, output_size: int, *, bias: bool):
        super().__init__()
        tp = PM.size_of("TP")
        if output_size % tp:
            raise ValueError(f"output_size={output_size} must be divisible by TP={tp}")
        self.weight = nn.Parameter(torch.empty(output_size // tp, input_size))
        self.bias = nn.Parameter(torch.zeros(output_size // tp)) if bias else None
        nn.init.xavier_uniform_(self.weight)
        set_tensor_model_parallel_attributes(self.weight, tp > 1, 0, 1)
        if self.bias is not None:
            set_tensor_model_parallel_attributes(self.bias, tp > 1, 0, 1)

    def forward(self, x):
        return _proj(x, self.weight, self.bias)


class TPRowLinear(nn.Module):
    def __init__(self, input_size: int, output_size: int, *, bias: bool, input_is_parallel: bool):
        super().__init__()
        tp = PM.size_of("TP")
        if input_size % tp:
            raise ValueError(f"input_size={input_size} must be divisible by TP={tp}")
        self.input_is_parallel = input_is_parallel
        self.weight = nn.Parameter(torch.empty(output_size, input_size // tp))
        self.bias = nn.Parameter(torch.zeros(output_size)) if bias else None
        nn.init.xavier_uniform_(self.weight)
        set_tensor_model_parallel_attributes(self.weight, tp > 1, 1, 1)

    def forward(self, x):
        if not self.input_is_parallel:
            x = mappings.scatter_to_tensor_model_parallel_region(x, "TP")
        y = mappings.reduce_from_tensor_model_parallel_region(_proj(x, self.weight, None), "TP")
        return y if self.bias is None else y + self.bias.to(y.dtype)


class VisionMLP(nn.Module):
    def __init__(self, cfg: VisionTransformerConfig):
        super().__init__()
        self.fc1 = TPColumnLinear(cfg.hidden_size, cfg.ffn_hidden_size, bias=True)
        self.fc2 = TPRowLinear(cfg.ffn_hidden_size, cfg.hidden_size, bias=True, input_is_parallel=True)

    def forward(self, x):
        return self.fc2(quick_gelu(self.fc1(x)))


class VisionAttention(nn.Module):
    def __init__(self, cfg: VisionTransformerConfig):
        super().__init__()
        tp = PM.size_of("TP")
        if cfg.hidden_size % cfg.num_attention_heads:
            raise ValueError("hidden_size must be divisible by num_attention_heads")
        if cfg.num_attention_heads % tp:
            raise ValueError(f"num_attention_heads={cfg.num_attention_heads} must be divisible by TP={tp}")
        self.num_local_heads = cfg.num_attention_heads // tp
        self.head_dim = cfg.hidden_size // cfg.num_attention_heads
        grid = cfg.image_size // cfg.patch_size
        self.rope = EncoderRope2D(self.head_dim, grid, grid, use_cls_token=cfg.use_cls_token, theta=cfg.rope_theta,
                                  theta_rescale_factor=cfg.rope_theta_rescale_factor) if cfg.use_rope2d else None
        self.attention_dropout = float(cfg.attention_dropout)
        self.qkv_proj = TPColumnLinear(cfg.hidden_size, cfg.hidden_size * 3, bias=True)
        self.out_proj = TPRowLinear(cfg.hidden_size, cfg.hidden_size, bias=True, input_is_parallel=True)

    def forward(self, x: torch.Tensor, grid_hw: tuple[int, int]) -> torch.Tensor:
        B, L, _ = x.shape
        h, D = self.num_local_heads, self.head_dim
        q, k, v = self.qkv_proj(x).reshape(B, L, 3, h, D).unbind(dim=2)
        if self.rope is not None:
            q, k = self.rope(q, k, grid_hw)
        if self.attention_dropout > 0.0 and self.training:
            # dropout on the attention probabilities is not part of the flash kernel: the library path is used
            o = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2),
                                               dropout_p=self.attention_dropout).transpose(1, 2)
            return self.out_proj(o.reshape(B, L, h * D))
        cu = torch.arange(0, (B + 1) * L, L, dtype=torch.int32, device=x.device)  # one segment per image
        fn = attention if (D == 128 and x.is_cuda) else attention_reference
        args = (q.reshape(B * L, h, D), k.reshape(B * L, h, D), v.reshape(B * L, h, D), cu, cu)
        o = fn(*args, L, causal=False) if fn is attention else fn(*args, causal=False)
        return self.out_proj(o.reshape(B, L, h * D))


class VisionBlock(nn.Module):
    def __init__(self, cfg: VisionTransformerConfig):
        super().__init__()
        ls = cfg.layer_scale_init_value
        self.ln_1 = nn.LayerNorm(cfg.hidden_size, eps=cfg.layernorm_epsilon)
        self.attn = VisionAttention(cfg)
        self.ls_1 = LayerScale(cfg.hidden_size, ls) if ls is not None else nn.Identity()
        self.ln_2 = nn.LayerNorm(cfg.hidden_size, eps=cfg.layernorm_epsilon)
        self.mlp = VisionMLP(cfg)
        self.ls_2 = LayerScale(cfg.hidden_size, ls) if ls is not None else nn.Identity()

    def forward(self, x, grid_hw):
        x = x + self.ls_1(self.attn(self.ln_1(x), grid_hw))
        return x + self.ls_2(self.mlp(self.ln_2(x)))


class VisionBackbone(nn.Module):
    def __init__(self, cfg: VisionTransformerConfig):
        super().__init__()
        self.resblocks = nn.ModuleList([VisionBlock(cfg) for _ in range(cfg.num_layers)])

    def forward(self, x, grid_hw):
        for blk in self.resblocks:
            x = blk(x, grid_hw)
        return x


class VisionTransformer(nn.Module):
    def __init__(self, cfg: VisionTransformerConfig):
        super().__init__()
        self.cfg = cfg
        self.conv1 = nn.Conv2d(cfg.in_channels, cfg.hidden_size, cfg.patch_size, stride=cfg.patch_size,
                               bias=cfg.patch_embed_bias)
        if cfg.use_cls_token:
            self.class_embedding = nn.Parameter(torch.randn(cfg.hidden_size))
        self.num_patches = (cfg.image_size // cfg.patch_size) ** 2
        self.positional_embedding = nn.Parameter(
            torch.randn(self.num_patches + (1 if cfg.use_cls_token else 0), cfg.hidden_size))
        self.ln_pre = nn.LayerNorm(cfg.hidden_size, eps=cfg.layernorm_epsilon) if cfg.use_ln_pre else nn.Identity()
        self.transformer = VisionBackbone(cfg)
        self.vit_downsampler1 = nn.Conv2d(cfg.hidden_size, cfg.vit_downsampler_hidden_dim,
                                          cfg.vit_downsampler1_kernel_size, stride=2,
                                          padding=cfg.vit_downsampler1_padding, bias=True)
        self.vit_downsampler2 = nn.Conv2d(cfg.vit_downsampler_hidden_dim, cfg.output_dim,
                                          cfg.vit_downsampler2_kernel_size, stride=2,
                                          padding=cfg.vit_downsampler2_padding, bias=True)

    def _patch_embed(self, pixel_values: torch.Tensor) -> torch.Tensor:
        """Non-overlapping patches: the convolution is ``unfold`` + one GEMM."""
        p = self.cfg.patch_size
        B, C, H, W = pixel_values.shape
        cols = F.unfold(pixel_values, kernel_size=p, stride=p).transpose(1, 2)          # [B, L, C*p*p]
        return _proj(cols, self.conv1.weight.reshape(self.conv1.out_channels, -1), self.conv1.bias)

    def _build_embeddings(self, pixel_values: torch.Tensor) -> torch.Tensor:
        x = self._patch_embed(pixel_values)
        if self.cfg.use_cls_token:
            cls = self.class_embedding.to(x.dtype).expand(x.shape[0], 1, -1)
            x = torch.cat([cls, x], dim=1)
        pe = interpolate_positional_embedding(self.positional_embedding.to(x.dtype), x.shape[1],
                                              use_cls_token=self.cfg.use_cls_token)
        return self.ln_pre(x + pe)

    def forward(self, pixel_values: torch.Tensor) -> torch.Tensor:
        """``[B, C, H, W]`` -> ``[B, tokens, output_dim]`` with ``tokens = (H / patch / 4) * (W / patch / 4)``."""
        p = self.cfg.patch_size
        x = self._build_embeddings(pixel_values)
        x = self.transformer(x, (pixel_values.shape[-2] // p, pixel_values.shape[-1] // p))
        if self.cfg.use_cls_token:
            x = x[:, 1:, :]
        B, L, H = x.shape
        side = math.isqrt(L)
        if side * side != L:
            raise ValueError(f"Expected square patch grid, got {L} tokens")
        x = x.transpose(1, 2).reshape(B, H, side, side)
        x = self.vit_downsampler2(self.vit_downsampler1(x))
        return x.flatten(2).transpose(1, 2)

    @property
    def reshaper(self):
        from ...checkpointing.reshape_ops import (MHA_TP_CHUNK, ColumnParallel, Duplicate, KeepThisTP, OnlineReshaper,
                                                  Rename, RowParallel, Script)

        def dup(name):
            return Script(src=name, op=Duplicate() + KeepThisTP(), dst=name)

        scripts = [dup("positional_embedding"), dup("conv1.weight"), dup("vit_downsampler1.*"), dup("vit_downsampler2.*")]
        if hasattr(self, "class_embedding"):
            scripts.insert(0, dup("class_embedding"))
        if self.conv1.bias is not None:
            scripts.append(dup("conv1.bias"))
        if not isinstance(self.ln_pre, nn.Identity):
            scripts += [dup("ln_pre.weight"), dup("ln_pre.bias")]
        for i in range(len(self.transformer.resblocks)):
            p = f"transformer.resblocks.{i}"
            scripts += [
                Script(src=f"{p}.attn.qkv_proj.*", op=MHA_TP_CHUNK() + KeepThisTP(), dst=f"{p}.attn.qkv_proj.*"),
                Script(src=f"{p}.attn.out_proj.weight", op=RowParallel() + KeepThisTP(), dst=f"{p}.attn.out_proj.weight"),
                dup(f"{p}.attn.out_proj.bias"), dup(f"{p}.ln_*.weight"), dup(f"{p}.ln_*.bias"), dup(f"{p}.ls_*.gamma"),
                Script(src=f"{p}.mlp.c_fc.*", op=ColumnParallel() + KeepThisTP() + Rename(f"{p}.mlp.fc1.*: {p}.mlp.c_fc.*"),
                       dst=f"{p}.mlp.fc1.*"),
                Script(src=f"{p}.mlp.c_proj.weight",
                       op=RowParallel() + KeepThisTP() + Rename(f"{p}.mlp.fc2.weight: {p}.mlp.c_proj.weight"),
                       dst=f"{p}.mlp.fc2.weight"),
                Script(src=f"{p}.mlp.c_proj.bias",
                       op=Duplicate() + KeepThisTP() + Rename(f"{p}.mlp.fc2.bias: {p}.mlp.c_proj.bias"),
                       dst=f"{p}.mlp.fc2.bias"),
            ]
        return OnlineReshaper(scripts)
