"""Datasets (reference ``steptronoss/data/datasets/*.py``): raw StepChat JSON conversations, and compiled
datasets (templated samples pickled into indexed-bin shards: sample ``i`` lives in shard ``i % n_shards`` at
local index ``i // n_shards``; ``compiled_dataset.pkl`` holds ``length``, ``shards`` and ``sample_meta``)."""
from __future__ import annotations

import json
import os
import pickle

from .indexed_bin import IndexedBinReader, IndexedBinWriter


class Dataset:
    def __len__(self) -> int:
        raise NotImplementedError

    def __getitem__(self, i: int) -> dict:
        raise NotImplementedError

    def sample_length(self, i: int) -> int:
        return len(self[i]["tokens"])


class StepChatJsonDataset(Dataset):
    """Top-level JSON list of ``{"conversations": [{role, content | [{type, value, loss_mask}], loss_mask, ...}]}``.
    Files are parsed with ``ijson`` when available (streaming), with ``json`` otherwise."""

    def __init__(self, paths, template=None):
        self.paths = [paths] if isinstance(paths, str) else list(paths)
        self.template = template
        self.records: list = []
        for p in self.paths:
            self.records.extend(self._read(p))

    @staticmethod
    def _read(path: str):
        try:
            import ijson

            with open(path, "rb") as f:
                return list(ijson.items(f, "item"))
        except ImportError:
            with open(path) as f:
                return json.load(f)

    def __len__(self) -> int:
        return len(self.records)

    def __getitem__(self, i: int) -> dict:
        rec = self.records[i]
        if self.template is None:
            return rec
        out = self.template(rec["conversations"])
        out["raw_index"] = i
        return out


def compile_dataset(dataset: Dataset, save_path: str, n_shards: int = 1, cfg: dict | None = None) -> dict:
    os.makedirs(save_path, exist_ok=True)
    writers = [IndexedBinWriter(os.path.join(save_path, f"shard_{s:05d}"), cfg=cfg) for s in range(n_shards)]
    meta = []
    for i in range(len(dataset)):
        sample = dataset[i]
        writers[i % n_shards].append(sample)
        meta.append(len(sample["tokens"]))
    for w in writers:
        w.close()
    manifest = {"length": len(dataset), "shards": [{"path": f"shard_{s:05d}", "size": len(range(s, len(dataset), n_shards))}
                                                    for s in range(n_shards)], "sample_meta": meta}
    with open(os.path.join(save_path, "compiled_dataset.pkl"), "wb") as f:
        pickle.dump(manifest, f)
    return manifest


class CompiledDataset(Dataset):
    def __init__(self, path: str):
        mf = os.path.join(path, "compiled_dataset.pkl")
        if not os.path.exists(mf):
            raise FileNotFoundError(f"manifest file not found: is '{path}' a compiled dataset?")
        with open(mf, "rb") as f:
            self.manifest = pickle.load(f)
        self.readers = [IndexedBinReader(os.path.join(path, s["path"])) for s in self.manifest["shards"]]

    def __len__(self) -> int:
        return self.manifest["length"]

    def __getitem__(self, i: int) -> dict:
        n = len(self.readers)
        return self.readers[i % n][i // n]

    def sample_length(self, i: int) -> int:
        return self.manifest["sample_meta"][i]
