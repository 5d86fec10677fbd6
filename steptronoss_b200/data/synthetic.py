"""Synthetic packed-document batches in the micro-batch contract of the framework.

One micro-batch is one packed sequence: ``input_ids [1,S]``, ``labels [1,S]`` (next token inside
each document), ``loss_masks [1,S]`` fp32, ``cu_seqlens [n_docs+1]`` int32, ``max_seq_len`` and
``position_id [S]`` int32 restarting at every document (the contract produced by the reference's
``SFTDataConfig.pack`` / ``preprocess``, ``playground/data/sft/oss260312/step_sft_data_config0311.py:193-286``).

Document lengths are uniform in ``[min_len, max_len]`` and are cut to fill the sequence exactly;
token ids are uniform over the vocabulary; the loss mask covers the second half of each document.
"""
from __future__ import annotations

import numpy as np
import torch

from ..config import Ref
from ..exp.base_exp import DataConfig
from ..utils.general import get_position_id_from_cu_seqlens


def make_packed_sample(rng: np.random.Generator, seq_len: int, vocab: int, min_len: int, max_len: int,
                       mask_second_half: bool = True) -> dict:
    lens = []
    left = seq_len
    while left > 0:
        ln = int(rng.integers(min_len, max_len + 1))
        ln = min(ln, left)
        lens.append(ln)
        left -= ln
    tokens = rng.integers(0, vocab, size=seq_len + 1, dtype=np.int64)
    ids = torch.from_numpy(tokens[:-1].copy())
    labels = torch.from_numpy(tokens[1:].copy())
    cu = torch.zeros(len(lens) + 1, dtype=torch.int32)
    cu[1:] = torch.cumsum(torch.tensor(lens, dtype=torch.int64), 0).to(torch.int32)
    mask = torch.zeros(seq_len, dtype=torch.float32)
    for i, ln in enumerate(lens):
        s, e = int(cu[i]), int(cu[i + 1])
        mask[(s + ln // 2 if mask_second_half else s) : e] = 1.0
        mask[e - 1] = 0.0  # the token after a document end belongs to the next document
    return {
        "input_ids": ids.unsqueeze(0),
        "labels": labels.unsqueeze(0),
        "loss_masks": mask.unsqueeze(0),
        "cu_seqlens": cu,
        "max_seq_len": torch.tensor(max(lens), dtype=torch.int32),
        "position_id": get_position_id_from_cu_seqlens(cu),
    }


class SyntheticPackedLoader:
    """Endless iterator of packed samples; deterministic per ``(seed, dp_rank)``; resumable.

    ``pin=True`` returns tensors in pinned host memory so that the trainer's host-to-device copy is
    asynchronous."""

    def __init__(self, seq_len: int, vocab: int, min_len: int = 256, max_len: int = 8192, seed: int = 0,
                 dp_rank: int = 0, dp_size: int = 1, pin: bool = False, length: int | None = None,
                 mask_second_half: bool = True):
        self.seq_len, self.vocab, self.min_len, self.max_len = seq_len, vocab, min_len, min(max_len, seq_len)
        self.seed, self.dp_rank, self.dp_size = seed, dp_rank, dp_size
        self.pin = pin and torch.cuda.is_available()
        self.index = 0
        self.length = length
        self.mask_second_half = mask_second_half

    def __len__(self) -> int:
        return self.length if self.length is not None else 1 << 40

    def __iter__(self):
        return self

    def __next__(self) -> dict:
        if self.length is not None and self.index * self.dp_size >= self.length:
            raise StopIteration
        global_index = self.index * self.dp_size + self.dp_rank
        rng = np.random.default_rng([self.seed, global_index])
        self.index += 1
        s = make_packed_sample(rng, self.seq_len, self.vocab, min(self.min_len, self.seq_len), self.max_len,
                               self.mask_second_half)
        if self.pin:
            s = {k: v.pin_memory() for k, v in s.items()}
        return s

    def state_dict(self) -> dict:
        # the position in the GLOBAL sample stream travels too, so that a job with another data-parallel size
        # continues with the sample that comes next
        return {"index": self.index, "consumed": self.index * self.dp_size}

    def load_state_dict(self, sd: dict) -> None:
        if "consumed" in sd:
            self.index = -(-int(sd["consumed"]) // self.dp_size)
        else:
            self.index = int(sd["index"])


class SyntheticDataConfig(DataConfig):
    """Synthetic packed documents of the experiment's sequence length and vocabulary."""

    seq_length = Ref("..trainer_cfg.global_seq_length", 8192)
    vocab_size = Ref("..model_cfg.tok_embed_cfg.vocab_size", 32000)
    min_doc_len: int = 256
    max_doc_len: int = 8192
    data_seed: int = 0
    num_samples: int | None = None
    pin_memory: bool = True
    global_data_keys: list | None = ["cu_seqlens", "position_id", "max_seq_len"]

    def build_dataloader(self, dp_rank: int = 0, dp_size: int = 1):
        return SyntheticPackedLoader(self.seq_length, self.vocab_size, self.min_doc_len, self.max_doc_len,
                                     self.data_seed, dp_rank, dp_size, self.pin_memory, self.num_samples)
