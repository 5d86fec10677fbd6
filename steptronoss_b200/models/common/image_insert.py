"""Vision features spliced into the token embeddings of a decoder.

Reference: ``steptronoss/model/common/parallel_embedding.py:84-205`` (``ImageForInsert``,
``ImageInsertEmbedding``) and ``steptronoss/model/common/image_insert_decoder.py:13-161`` (the decoder mixin
that runs the vision encoder under its own mesh through a :class:`MeshConnector`).

Flow on the first pipeline stage: raw images -> ``MeshConnector.forward`` (to the encoder's mesh) -> vision
encoder -> ``MeshConnector.backward`` (features back on every text rank) -> linear projector to the hidden
size -> the features of image ``i`` overwrite the embeddings that follow the ``i``-th start token.
Embeddings are token-major ``[tokens, H]``; with sequence parallelism the splice happens on the full
sequence and the result is then scattered over TP.
"""
from __future__ import annotations

import torch

from ...config import DataClass
from ...parallel import mappings
from ...parallel.state import PM
from ...utils.logger import logger
from .mesh_connector import MeshConnector
from .parallel_embedding import InputEmbeddingConfig, WordEmbedding
from .vit import VisionTransformerConfig


class ImageForInsert(DataClass):
    insert_start_token: int = None
    """token id after which the visual features are inserted"""
    images: torch.Tensor | None = None
    """raw images ``[N, 3, H, W]``"""
    image_features: torch.Tensor | list | None = None
    """encoder output (before the language projector), ``[N, L, C]`` or a list of ``[L, C]``"""
    rope_cu_seqlens: torch.Tensor | None = None
    rope_max_seq_len: int | None = None


class ImageInsertInputEmbeddingConfig(InputEmbeddingConfig):
    encoder_cfg: VisionTransformerConfig = VisionTransformerConfig
    img_start_token: int = 0
    encoder_no_grad: bool = False
    projector_bias: bool = False

    def build_adapter(self) -> torch.nn.Module:
        lin = torch.nn.Linear(self.encoder_cfg.output_dim, self.hidden_size, bias=self.projector_bias)
        torch.nn.init.kaiming_normal_(lin.weight, mode="fan_in", nonlinearity="relu")
        if lin.bias is not None:
            torch.nn.init.zeros_(lin.bias)
        return lin

    def build_model(self):
        return ImageInsertEmbedding(self)


class ImageInsertEmbedding(WordEmbedding):
    def __init__(self, cfg: ImageInsertInputEmbeddingConfig):
        super().__init__(cfg)
        self.align_projector = cfg.build_adapter().to(self.word_embeddings.weight.device)
        self.align_projector.weight.has_initialized = True  # keeps its own initialisation

    @staticmethod
    def _feature_list(feats, device, dtype) -> list:
        if torch.is_tensor(feats):
            if feats.dim() != 3:
                raise ValueError(f"Expected image_features with shape [N, L, C], got {tuple(feats.shape)}")
            out = list(feats.unbind(0))
        else:
            out = []
            for f in feats:
                if f.dim() == 3:
                    out.extend(f.unbind(0))
                elif f.dim() == 2:
                    out.append(f)
                else:
                    raise ValueError(f"Expected feature tensor rank 2 or 3, got rank {f.dim()}")
        return [f.to(device=device, dtype=dtype) for f in out]

    @staticmethod
    def insert_features(emb: torch.Tensor, feats, input_ids: torch.Tensor, flag: int) -> torch.Tensor:
        """``emb [tokens, H]``: rows after the i-th occurrence of ``flag`` are replaced by the i-th feature."""
        feats = ImageInsertEmbedding._feature_list(feats, emb.device, emb.dtype)
        if not feats:
            return emb
        starts = (torch.nonzero(input_ids.reshape(-1) == flag, as_tuple=False).reshape(-1) + 1).tolist()
        if len(starts) != len(feats):
            logger.warning(f"Mismatch between image features and insert locations: {len(feats)} features vs "
                           f"{len(starts)} locations; truncating to the overlap.")
        pieces, cursor = [], 0
        for start, f in zip(starts, feats):
            end = min(start + f.shape[0], emb.shape[0])
            if end <= start or start < cursor:
                continue
            pieces += [emb[cursor:start], f[: end - start]]
            cursor = end
        pieces.append(emb[cursor:])
        return torch.cat(pieces, dim=0)  # differentiable w.r.t. both the embeddings and the features

    def forward(self, input_ids: torch.Tensor, images: list | None = None, **kw) -> torch.Tensor:
        ids = input_ids.reshape(-1)
        if not images:
            return super().forward(ids)
        we = self.word_embeddings
        sp = we.sequence_parallel
        from ...ops.fused import embedding  # noqa: F401  (same op the table uses)

        full = embedding(ids, we.weight, we.vocab_start, we.vocab_end)
        full = mappings.reduce_from_tensor_model_parallel_region(full, we.group)
        if full.dtype != self.cfg.params_dtype and not self.cfg.fp32_residual_connection:
            full = full.to(self.cfg.params_dtype)
        w = self.align_projector.weight
        for im in images:
            if im.image_features is None:
                raise ValueError("ImageInsertEmbedding expects precomputed image_features in decoupled-encoder mode")
            f = im.image_features
            proj = (self.align_projector(f.to(device=w.device, dtype=w.dtype)) if torch.is_tensor(f)
                    else [self.align_projector(x.to(device=w.device, dtype=w.dtype)) for x in f])
            full = self.insert_features(full, proj, ids, im.insert_start_token)
        return mappings.scatter_to_sequence_parallel_region(full, we.group) if sp else full


class ImageInsertDecoderMixin:
    """Mix into a decoder model whose ``tok_embed_cfg`` is an :class:`ImageInsertInputEmbeddingConfig`; call
    ``build_multimodal_modules()`` at the end of ``__init__``."""

    def build_multimodal_modules(self) -> None:
        enc_cfg = self.cfg.tok_embed_cfg.encoder_cfg
        dev = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
        with PM.use_mesh(enc_cfg.parallel_cfg):
            self.encoder = enc_cfg.build_model().to(device=dev, dtype=self.cfg.params_dtype)
        for p in self.encoder.parameters():
            p.has_initialized = True  # the encoder keeps its own initialisation
            if self.cfg.tok_embed_cfg.encoder_no_grad:
                p.requires_grad = False
        self.mesh_connector = MeshConnector(self.cfg.parallel_cfg, enc_cfg.parallel_cfg,
                                            is_data_source=self.is_first_stage, dup_dim=["TP"])

    # ------------------------------------------------------------------ HF <-> native weights
    # The text model's mapping (an attribute that its constructor assigns, or its ``build_reshaper``) is kept as it
    # is; the vision encoder and the projector add their rules in front of it.  HF spelling: ``vision_model.*`` with
    # torch's fused ``in_proj_weight / in_proj_bias`` for the attention input projection, and
    # ``vit_large_projector.weight`` (reference ``steptronoss/model/common/image_insert_decoder.py:52-96``).
    @property
    def reshaper(self):
        from ...checkpointing.reshape_ops import OnlineReshaper

        base = self.__dict__.get("_text_reshaper")
        if base is None and hasattr(super(), "build_reshaper"):
            base = super().build_reshaper()
        if base is None or "encoder" not in self._modules:
            return base
        return OnlineReshaper(self.multimodal_reshape_scripts() + list(base.scripts))

    @reshaper.setter
    def reshaper(self, value):
        self.__dict__["_text_reshaper"] = value

    def multimodal_reshape_scripts(self) -> list:
        from ...checkpointing.reshape_ops import Duplicate, KeepThisTP, Prefixed, Rename, Script

        if not self.is_first_stage:          # one pipeline stage exports the vision weights
            return []
        scripts = []
        proj = getattr(getattr(self, "tok_embeddings", None), "align_projector", None)
        if proj is not None:
            for leaf in ("weight", "bias") if proj.bias is not None else ("weight",):
                scripts.append(Script(src=f"vit_large_projector.{leaf}", dst=f"tok_embeddings.align_projector.{leaf}",
                                      op=Duplicate() + KeepThisTP()
                                      + Rename(f"tok_embeddings.align_projector.{leaf}: vit_large_projector.{leaf}")))
        if hasattr(self.encoder, "reshaper"):
            fused = [("*.attn.in_proj_weight", "*.attn.qkv_proj.weight"), ("*.attn.in_proj_bias", "*.attn.qkv_proj.bias")]
            scripts.append(Script(src="vision_model.*", dst="encoder.*",
                                  op=Prefixed(self.encoder.reshaper, "vision_model.", "encoder.", fused,
                                              mesh=self.cfg.tok_embed_cfg.encoder_cfg.parallel_cfg)))
        return scripts

    def _encode_images_for_insert(self, images: list | None) -> list | None:
        if not images:
            return images
        p0 = next(self.encoder.parameters())
        enc_cfg = self.cfg.tok_embed_cfg.encoder_cfg
        out = []
        for im in images:
            if im.image_features is not None:
                out.append(im)
                continue
            if im.images is None:
                raise ValueError("ImageForInsert requires either images or image_features")
            local = self.mesh_connector.forward(im.images)
            feats = None
            if local is not None:
                if local.shape[0] == 0:
                    feats = local.new_empty((0, 0, 0))
                else:
                    with PM.use_mesh(enc_cfg.parallel_cfg), \
                            torch.set_grad_enabled(not self.cfg.tok_embed_cfg.encoder_no_grad and torch.is_grad_enabled()):
                        feats = self.encoder(local.to(device=p0.device, dtype=p0.dtype))
            feats = self.mesh_connector.backward(feats)
            out.append(ImageForInsert(insert_start_token=im.insert_start_token, image_features=feats,
                                      rope_cu_seqlens=im.rope_cu_seqlens, rope_max_seq_len=im.rope_max_seq_len))
        return out

    def forward_head(self, input_ids=None, images=None, **data):
        emb = self.tok_embeddings(input_ids, images=self._encode_images_for_insert(images))
        if PM.size_of("CP") > 1:
            from ...parallel.context_parallel import scatter_to_balanced_cp_region

            emb = scatter_to_balanced_cp_region(emb, dim=0)
        return emb
