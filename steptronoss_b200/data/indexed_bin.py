"""Indexed binary shards (reference ``steptronoss/data/utils/indexed_bin_file.py:78-358``).

A shard directory holds ``data.bin`` (concatenated pickled records), ``index.npz`` (``offsets`` and ``sizes``
as little-endian uint64), an optional ``cfg.json`` and a ``.success`` marker written last.  Readers use
``os.pread`` so that forked workers can share one descriptor."""
from __future__ import annotations

import json
import os
import pickle

import numpy as np


class IndexedBinWriter:
    def __init__(self, path: str, cfg: dict | None = None):
        self.path = path
        os.makedirs(path, exist_ok=True)
        self._f = open(os.path.join(path, "data.bin"), "wb")
        self._offsets, self._sizes, self._pos = [], [], 0
        self._cfg = cfg

    def append(self, record) -> int:
        blob = pickle.dumps(record, protocol=pickle.HIGHEST_PROTOCOL)
        self._f.write(blob)
        self._offsets.append(self._pos)
        self._sizes.append(len(blob))
        self._pos += len(blob)
        return len(self._offsets) - 1

    def close(self) -> None:
        self._f.close()
        np.savez(os.path.join(self.path, "index.npz"), offsets=np.asarray(self._offsets, dtype="<u8"),
                 sizes=np.asarray(self._sizes, dtype="<u8"))
        if self._cfg is not None:
            with open(os.path.join(self.path, "cfg.json"), "w") as f:
                json.dump(self._cfg, f)
        open(os.path.join(self.path, ".success"), "w").close()

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()


class IndexedBinReader:
    def __init__(self, path: str):
        if not os.path.exists(os.path.join(path, ".success")):
            raise FileNotFoundError(f"{path} is not a complete indexed-bin shard (.success missing)")
        idx = np.load(os.path.join(path, "index.npz"))
        self.offsets, self.sizes = idx["offsets"], idx["sizes"]
        self._fd = os.open(os.path.join(path, "data.bin"), os.O_RDONLY)

    def __len__(self) -> int:
        return len(self.offsets)

    def __getitem__(self, i: int):
        return pickle.loads(os.pread(self._fd, int(self.sizes[i]), int(self.offsets[i])))

    def close(self) -> None:
        if self._fd is not None:
            os.close(self._fd)
            self._fd = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
