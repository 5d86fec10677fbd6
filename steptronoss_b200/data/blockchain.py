"""A portable chain of pickled blocks for moving and feeding samples
(reference ``steptronoss/data/utils/blockchain.py:11-349``).

``root.pkl`` is an empty block whose ``next`` names the first data block and its checksum; every block names
its successor, so a directory can be copied while it is still being appended to.  ``Chain.writer`` appends
blocks of ``block_size`` samples; ``Chain.get`` iterates them (wrapping around to the first block at the
end, as a training stream does), optionally prefetching blocks on a thread; ``state_dict`` is the position.
"""
from __future__ import annotations

import contextlib
import os
import pickle
import threading
import time
from hashlib import md5

from ..utils.logger import logger


class Block:
    def __init__(self, root: str = "", target_file: str | None = None, checksum: str = "EMPTY", next=None,
                 verify: bool = True):
        self.root, self.target_file, self.checksum, self.verify = root, target_file, checksum, verify
        self.next = list(next) if next else [None, "EMPTY"]
        self.data: list = []
        self.loaded = False
        if root and target_file and not os.path.exists(self.target_path):
            os.makedirs(root, exist_ok=True)
            self.save()

    @property
    def target_path(self) -> str:
        return os.path.join(self.root, self.target_file)

    def md5(self) -> str:
        return md5(pickle.dumps(self.data)).hexdigest()

    def load(self) -> None:
        with open(self.target_path, "rb") as f:
            self.data, self.next = pickle.load(f)
        if self.verify and self.data and self.checksum not in ("EMPTY", ""):
            now = self.md5()
            if now != self.checksum:
                logger.warning(f"Checksum mismatch on {self.target_path}. Double check if this is expected.")
                self.checksum = now
        self.loaded = True

    def unload(self) -> None:
        self.data, self.loaded = [], False

    def save(self, file: str | None = None) -> None:
        if file:
            self.target_file = file
        tmp = self.target_path + ".tmp"
        with open(tmp, "wb") as f:
            pickle.dump([self.data, self.next], f)
        os.replace(tmp, self.target_path)

    def __len__(self) -> int:
        return len(self.data)

    def state_dict(self) -> dict:
        return {"target_file": self.target_file, "checksum": self.checksum, "next": self.next}


class Chain:
    def __init__(self, root: str = "", verify: bool = True, prefetch: int = 0, verbose: bool = False):
        self.root, self.verify, self.prefetch, self.verbose = root, verify, prefetch, verbose
        self.blocks: list = [Block(root, "root.pkl", verify=verify)]
        self.block_id, self.in_block_id = 0, 0
        self._loader: threading.Thread | None = None
        self._stop = False
        self._lock = threading.RLock()  # the prefetch thread and the reader both extend / load the block list

    # ------------------------------------------------------------------ writing
    @contextlib.contextmanager
    def writer(self, block_size: int = 1000):
        """``with chain.writer(1000) as write: write(sample)`` appends after the current last block."""
        last = self._walk_to_end()
        buf: list = []
        index = [len(self._all_files())]

        def flush():
            nonlocal last
            if not buf:
                return
            blk = Block(verify=self.verify)
            blk.root, blk.data = self.root, list(buf)
            digest = blk.md5()
            blk.target_file = f"block_{index[0]}_{digest[:8]}.pkl"
            blk.checksum = digest
            blk.save()
            last.load() if not last.loaded else None
            last.next = [blk.target_file, digest]
            last.save()
            last, index[0] = blk, index[0] + 1
            blk.loaded = True
            buf.clear()

        def write(sample):
            buf.append(sample)
            if len(buf) >= block_size:
                flush()

        try:
            yield write
        finally:
            flush()

    def _all_files(self) -> list:
        return [f for f in os.listdir(self.root) if f.startswith("block_")] if os.path.isdir(self.root) else []

    def _walk_to_end(self) -> Block:
        blk = self.blocks[0]
        blk.load()
        while blk.next and blk.next[0] is not None:
            blk = Block(self.root, blk.next[0], blk.next[1], verify=False)
            blk.load()
        return blk

    # ------------------------------------------------------------------ reading
    def _block(self, i: int) -> Block | None:
        with self._lock:
            return self._block_locked(i)

    def _block_locked(self, i: int) -> Block | None:
        while i >= len(self.blocks):
            tail = self.blocks[-1]
            if not tail.loaded:
                tail.load()
            if tail.next[0] is None:
                return None
            self.blocks.append(Block(self.root, tail.next[0], tail.next[1], verify=self.verify))
        blk = self.blocks[i]
        if not blk.loaded:
            if self.verbose:
                logger.info(f"FetchBlock -> {blk.target_file}")
            blk.load()
        return blk

    def _prefetch_loop(self):
        while not self._stop:
            for ahead in range(1, self.prefetch + 1):
                try:
                    self._block(self.block_id + ahead)
                except Exception:
                    break
            time.sleep(0.05)

    def get(self):
        """Next sample; after the last block the chain restarts from the first one. ``None`` for an empty chain."""
        if self.prefetch and self._loader is None:
            self._loader = threading.Thread(target=self._prefetch_loop, daemon=True)
            self._loader.start()
        for _ in range(2):
            blk = self._block(self.block_id)
            while blk is not None and self.in_block_id >= len(blk):
                if self.block_id > 1:
                    with self._lock:
                        self.blocks[self.block_id - 1].unload()
                self.block_id, self.in_block_id = self.block_id + 1, 0
                blk = self._block(self.block_id)
            if blk is not None:
                item = blk.data[self.in_block_id]
                self.in_block_id += 1
                return item
            if len(self.blocks) <= 1:
                return None
            logger.warning(f"{len(self.blocks)=}. next_block is empty, restart from root!!!")
            self.block_id, self.in_block_id = 0, 0
        return None

    def __iter__(self):
        return self

    def __next__(self):
        item = self.get()
        if item is None:
            raise StopIteration
        return item

    def state_dict(self) -> dict:
        return {"block_id": self.block_id, "in_block_id": self.in_block_id}

    def load_state_dict(self, state: dict) -> None:
        self.block_id, self.in_block_id = state["block_id"], state["in_block_id"]

    def close(self) -> None:
        self._stop = True
