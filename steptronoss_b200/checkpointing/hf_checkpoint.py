"""HF safetensors import and export (reference ``steptronoss/checkpointing/hf_checkpoint.py:56-122``,
``utils/weight_loader.py:34-364``).

Export: every pipeline chunk converts its parameters back to HF names (gathering TP / EP shards) and
the first TP ∧ DP rank of the chunk writes ``model-%05d.safetensors``; rank 0 writes
``model.safetensors.index.json`` and copies ``*.json`` / tokenizer files from ``config_source``.
"""
from __future__ import annotations

import glob
import json
import os
import shutil


from ..models.module import unwrap_model
from ..parallel.state import PM
from ..utils.dist_utils import all_gather_object


class HFWeights:
    """Lazy dict over the tensors of a HF checkpoint directory (sharded or single file)."""

    def __init__(self, path: str, device: str = "cpu", rename: dict | None = None):
        from safetensors import safe_open

        self.path, self.device = path, device
        self._where: dict[str, str] = {}
        index = os.path.join(path, "model.safetensors.index.json")
        if os.path.exists(index):
            for k, f in json.load(open(index))["weight_map"].items():
                self._where[k] = os.path.join(path, f)
        else:
            for f in sorted(glob.glob(os.path.join(path, "*.safetensors"))):
                with safe_open(f, framework="pt") as h:
                    for k in h.keys():
                        self._where[k] = f
        self._rename = rename or {}
        for new, old in list(self._rename.items()):
            if old in self._where:
                self._where[new] = self._where.pop(old)
        self._open = safe_open

    def keys(self):
        return self._where.keys()

    def __iter__(self):
        return iter(self._where)

    def __len__(self):
        return len(self._where)

    def __contains__(self, k):
        return k in self._where

    def __getitem__(self, k):
        f = self._where[k]
        src = self._rename.get(k, k)
        with self._open(f, framework="pt", device=self.device) as h:
            return h.get_tensor(src)

    def items(self):
        for k in self._where:
            yield k, self[k]


def load_safetensors_into(model, path: str, strict: bool = True) -> list:
    return model.load_hf_state_dict(HFWeights(path), strict=strict)


def dump_safetensors(models, out_dir: str, config_source: str | None = None) -> None:
    from safetensors.torch import save_file

    os.makedirs(out_dir, exist_ok=True)
    weight_map = {}
    for vp, m in enumerate(models):
        um = unwrap_model(m)
        hf = um.hf_state_dict()  # collective: gathers TP / EP shards
        chunk = um.pp_rank
        fname = f"model-{chunk + 1:05d}.safetensors"
        if PM.rank_in("TP") == 0 and PM.rank_in("DP") == 0:
            save_file({k: v.detach().cpu().contiguous() for k, v in hf.items()}, os.path.join(out_dir, fname))
            weight_map.update({k: fname for k in hf})
    merged: dict = {}
    for d in all_gather_object(weight_map):
        merged.update(d)
    if PM.world_rank == 0:
        with open(os.path.join(out_dir, "model.safetensors.index.json"), "w") as f:
            json.dump({"metadata": {}, "weight_map": merged}, f, indent=1)
        if config_source and os.path.isdir(config_source):
            for pat in ("*.json", "tokenizer*", "*.txt", "*.model"):
                for src in glob.glob(os.path.join(config_source, pat)):
                    if not src.endswith(".safetensors.index.json"):
                        shutil.copy(src, out_dir)
    PM.barrier()
