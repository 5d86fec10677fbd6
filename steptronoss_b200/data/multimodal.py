"""Helpers that turn the output of multimodal data transforms into model inputs (reference
``steptronoss/data/multimodal.py:9-101``)."""
from __future__ import annotations

from collections.abc import Callable, Iterable, Sequence

import torch

IMAGE_ITEM_TYPE = 0
PATCH_ITEM_TYPE = 1


def build_image_for_insert(images_and_types: Iterable, *, patch_start_id: int, image_start_id: int,
                           limit_images: int | None = None, limit_patches: int | None = None,
                           rope_args_fn: Callable | None = None, dtype: torch.dtype | None = torch.bfloat16,
                           to_cuda: bool = True) -> list:
    """``[(tensor, IMAGE_ITEM_TYPE | PATCH_ITEM_TYPE), ...]`` -> one ``ImageForInsert`` for the patches and
    one for the whole images (each stacked along dim 0), in that order."""
    from ..models.common.image_insert import ImageForInsert

    images, patches = [], []
    for t, kind in images_and_types:
        if kind == IMAGE_ITEM_TYPE:
            images.append(t)
        elif kind == PATCH_ITEM_TYPE:
            patches.append(t)
        else:
            raise ValueError(f"Unsupported multimodal image type: {kind}")
    images = images if limit_images is None else images[: int(limit_images)]
    patches = patches if limit_patches is None else patches[: int(limit_patches)]
    out = []
    for start, tensors in ((patch_start_id, patches), (image_start_id, images)):
        if not tensors:
            continue
        stacked = torch.stack(list(tensors), dim=0)
        if dtype is not None:
            stacked = stacked.to(dtype)
        if to_cuda and torch.cuda.is_available():
            stacked = stacked.to("cuda", non_blocking=True)
        extra = {}
        if rope_args_fn is not None:
            cu, mx = rope_args_fn(tensors)
            extra = {"rope_cu_seqlens": cu, "rope_max_seq_len": int(mx)}
        out.append(ImageForInsert(insert_start_token=start, images=stacked, **extra))
    return out


def compute_rope_args(images: Sequence, patch_size: int, *, to_cuda: bool = True):
    """Per-image patch counts as ``cu_seqlens`` (int32) and their maximum."""
    if not images:
        raise ValueError("images must be non-empty when computing RoPE args")
    counts = [(int(im.shape[-2]) // patch_size) * (int(im.shape[-1]) // patch_size) for im in images]
    cu = torch.zeros(len(counts) + 1, dtype=torch.int32)
    cu[1:] = torch.cumsum(torch.tensor(counts, dtype=torch.int32), dim=0)
    if to_cuda and torch.cuda.is_available():
        cu = cu.to("cuda")
    return cu, max(counts)
