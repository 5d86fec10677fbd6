"""Token permutation helpers with the Transformer-Engine style interface used by dispatcher back ends
(reference ``steptronoss/model/utils/permute_utils.py:129-277``).

Two routing descriptions are understood: ``"mask"`` - ``routing_map [tokens, experts]`` (bool/int): rows are
emitted expert-major, token order inside an expert; ``"index"`` - ``routing_map [tokens, top_k]`` of expert
indices: rows are emitted sorted by expert, stable.  ``row_id_map`` records, for every output row, the flat
source position (``expert * tokens + token`` for masks, ``token * top_k + k`` for indices; ``-1`` = padding)
and is what :func:`moe_unpermute` needs to send rows home (optionally weighted by ``merging_probs``).
"""
from __future__ import annotations

import torch


def _fit(indices: torch.Tensor, num_out_tokens: int) -> torch.Tensor:
    """Trim to ``num_out_tokens`` rows or pad with -1 (``num_out_tokens <= 0`` keeps everything)."""
    if num_out_tokens is None or num_out_tokens <= 0 or indices.numel() == num_out_tokens:
        return indices
    if indices.numel() > num_out_tokens:
        return indices[:num_out_tokens]
    pad = torch.full((num_out_tokens - indices.numel(),), -1, dtype=indices.dtype, device=indices.device)
    return torch.cat([indices, pad])


def _take_rows(inp: torch.Tensor, rows: torch.Tensor) -> torch.Tensor:
    out = inp.index_select(0, rows.clamp_min(0))
    return torch.where((rows >= 0).view(-1, *([1] * (inp.dim() - 1))), out, torch.zeros((), dtype=inp.dtype, device=inp.device))


def moe_permute(inp, routing_map, num_out_tokens: int = -1, max_token_num: int = -1, map_type: str = "mask"):
    out, row_id_map, _ = _permute(inp, routing_map, num_out_tokens, None, map_type)
    return out, row_id_map


def moe_permute_with_probs(inp, probs, routing_map, num_out_tokens: int = -1):
    out, row_id_map, p = _permute(inp, routing_map, num_out_tokens, probs, "mask")
    return out, p, row_id_map


def _permute(inp, routing_map, num_out_tokens, probs, map_type):
    T = inp.shape[0]
    if map_type == "mask":
        mask_t = routing_map.t().bool()                                   # [E, T]
        flat = mask_t.reshape(-1).nonzero(as_tuple=False).reshape(-1)     # expert-major, token order
        row_id_map = _fit(flat, num_out_tokens)
        tokens = torch.where(row_id_map >= 0, row_id_map % T, row_id_map)
        p = None
        if probs is not None:
            p = _take_rows(probs.t().reshape(-1), row_id_map)
        return _take_rows(inp, tokens), row_id_map, p
    if map_type == "index":
        K = routing_map.shape[1] if routing_map.dim() > 1 else 1
        flat_exp = routing_map.reshape(-1)
        order = torch.sort(flat_exp, stable=True).indices
        order = order[flat_exp[order] >= 0]
        row_id_map = _fit(order, num_out_tokens)
        tokens = torch.where(row_id_map >= 0, row_id_map // K, row_id_map)
        return _take_rows(inp, tokens), row_id_map, None
    raise ValueError("map_type should be one of 'mask' or 'index'")


def moe_unpermute(inp, row_id_map, merging_probs=None, restore_shape=None, map_type: str = "mask", probs=None):
    if probs is not None:
        if merging_probs is not None:
            raise ValueError("Both merging_probs and probs are provided. probs is deprecated.")
        merging_probs = probs
    if inp.numel() == 0:
        return inp
    if map_type not in ("mask", "index"):
        raise ValueError("map_type should be one of 'mask' or 'index'")
    if merging_probs is not None:
        T, K = merging_probs.shape
    elif restore_shape is not None:
        T, K = restore_shape[0], None
    elif map_type == "index":
        T, K = row_id_map.size(0), 1
    else:
        raise ValueError("restore_shape or merging_probs must be provided for map_type='mask'.")
    out = inp.new_zeros(restore_shape if restore_shape is not None else (T, inp.size(1)))
    valid = row_id_map >= 0
    ids = row_id_map[valid].long()
    rows = inp[valid]
    if map_type == "mask":
        tokens = ids % T
        w = merging_probs.t().reshape(-1).index_select(0, ids) if merging_probs is not None else None
    else:
        if K is None:
            K = int(ids.max()) // max(T, 1) + 1 if ids.numel() else 1
        tokens = ids // K
        w = merging_probs.reshape(-1).index_select(0, ids) if merging_probs is not None else None
    if w is not None:
        rows = rows * w.unsqueeze(-1).to(rows.dtype)
    return out.index_add(0, tokens, rows)


def moe_sort_chunks_by_index(inp, split_sizes, sorted_index):
    if inp.numel() == 0:
        return inp
    if split_sizes.dim() != 1 or sorted_index.dim() != 1:
        raise ValueError("split_sizes and sorted_index must be 1D")
    chunks = inp.split(split_sizes.tolist(), dim=0)
    picked = [chunks[i] for i in sorted_index.tolist()]
    return torch.cat(picked, dim=0) if picked else inp.new_empty((0, *inp.shape[1:]))


def moe_sort_chunks_by_index_with_probs(inp, probs, split_sizes, sorted_index):
    if inp.numel() == 0:
        return inp, probs
    if probs.size(0) != inp.size(0):
        raise ValueError("probs and inp must have the same leading dimension")
    return (moe_sort_chunks_by_index(inp, split_sizes, sorted_index),
            moe_sort_chunks_by_index(probs, split_sizes, sorted_index))
