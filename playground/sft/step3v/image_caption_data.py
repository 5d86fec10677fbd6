"""Image-caption SFT data for the vision-language models (stands where the reference reads Flickr8k through a HF
processor, ``playground/sft/step3v/step3v_flickr8k_data.py``).

``captions_file`` is a jsonl of ``{"image": "relative/path.jpg", "caption": "..."}`` next to the images.  A sample is
one user turn (image + instruction) and one assistant turn (the caption): the image is resized to the encoder's
resolution, one image start token is followed by as many placeholder tokens as the encoder emits features, and the
loss covers the caption tokens.  One sample per micro-batch, padded to ``max_seq_len``.
"""
from __future__ import annotations

import json
import os

import numpy as np
import torch

from steptronoss_b200.config import Ref
from steptronoss_b200.data.nextable import Nextable
from steptronoss_b200.exp.sft import SFTDataConfig


class CaptionStream(Nextable):
    def __init__(self, cfg: "ImageCaptionDataConfig", dp_rank: int, dp_size: int):
        super().__init__()
        self.cfg, self.pos, self.stride = cfg, dp_rank, dp_size
        self.rows = cfg.load_rows()
        self.tok = cfg.build_tokenizer()

    def __next__(self) -> dict:
        row = self.rows[self.pos % len(self.rows)]
        self.pos += self.stride
        return self.cfg.encode(self.tok, row)

    def state_dict(self) -> dict:
        return {"pos": self.pos}

    def load_state_dict(self, sd: dict) -> None:
        self.pos = sd["pos"]


class ImageCaptionDataConfig(SFTDataConfig):
    captions_file: str = os.environ.get("STB200_CAPTIONS", "./captions.jsonl")
    instruction: str = "Describe this image in one sentence."
    max_seq_len: int = 2048
    image_size = Ref("..model_cfg.tok_embed_cfg.encoder_cfg.image_size", 728)
    patch_size = Ref("..model_cfg.tok_embed_cfg.encoder_cfg.patch_size", 14)
    img_start_token = Ref("..model_cfg.tok_embed_cfg.img_start_token", 0)
    image_token_id = Ref("..model_cfg.tok_embed_cfg.image_token_id", 0)
    build_tokenizer = Ref("..tokenizer_cfg.build_tokenizer")
    global_data_keys = ["cu_seqlens", "position_id"]

    def load_rows(self) -> list:
        with open(self.captions_file, encoding="utf-8") as f:
            rows = [json.loads(line) for line in f if line.strip()]
        if not rows:
            raise ValueError(f"{self.captions_file} holds no samples")
        root = os.path.dirname(os.path.abspath(self.captions_file))
        return [{"image": os.path.join(root, r["image"]), "caption": r["caption"]} for r in rows]

    def features_per_image(self) -> int:
        side = self.image_size // self.patch_size // 4      # two stride-2 down-samplers
        return side * side

    def load_image(self, path: str) -> torch.Tensor:
        from PIL import Image

        img = Image.open(path).convert("RGB").resize((self.image_size, self.image_size))
        x = torch.from_numpy(np.asarray(img, dtype=np.float32) / 255.0).permute(2, 0, 1)
        mean = torch.tensor([0.485, 0.456, 0.406]).view(3, 1, 1)
        std = torch.tensor([0.229, 0.224, 0.225]).view(3, 1, 1)
        return (x - mean) / std

    def encode(self, tok, row: dict) -> dict:
        user = tok.encode(f"<|im_start|>user\n", add_special_tokens=False)
        image_slots = [self.img_start_token] + [self.image_token_id] * self.features_per_image()
        ask = tok.encode(f"\n{self.instruction}<|im_end|>\n<|im_start|>assistant\n", add_special_tokens=False)
        answer = tok.encode(f"{row['caption']}<|im_end|>\n", add_special_tokens=False)
        tokens = user + image_slots + ask + answer
        mask = [0.0] * (len(tokens) - len(answer)) + [1.0] * len(answer)
        tokens, mask = tokens[: self.max_seq_len + 1], mask[: self.max_seq_len + 1]
        batch = self.pack([{"tokens": np.asarray(tokens, dtype=np.int64), "loss_mask": np.asarray(mask, dtype=np.float32)}])
        batch["images"] = self.load_image(row["image"]).unsqueeze(0)
        return batch

    def build_dataloader(self, dp_rank: int = 0, dp_size: int = 1):
        return CaptionStream(self, dp_rank, dp_size)

    def preprocess(self, batch: dict) -> dict:
        from steptronoss_b200.models.common.image_insert import ImageForInsert

        out = super().preprocess(batch)
        if "images" in batch:
            dev = out["cu_seqlens"].device
            out["images"] = [ImageForInsert(insert_start_token=self.img_start_token,
                                            images=batch["images"].to(dev, non_blocking=True))]
        return out
