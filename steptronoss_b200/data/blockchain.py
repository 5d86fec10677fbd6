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
    def __init__(self, root: str = "", verify: bool = True, prefetch: int = 0, verbose: bool = False,
                 reusable: bool = False):
        """``reusable``: blocks stay in memory after they were read (a small chain that is iterated many times);
        otherwise a block is released once the reader is two blocks past it."""
        self._root, self.verify, self.prefetch, self.verbose, self.reusable = root, verify, prefetch, verbose, reusable
        self.blocks: list = [Block(root, "root.pkl", verify=verify)]
        self.block_id, self.in_block_id = 0, 0
        self._loader: threading.Thread | None = None
        self._stop = False
        self._lock = threading.RLock()  # the prefetch thread and the reader both extend / load the block list

    @property
    def root(self) -> str:
        return self._root

    @root.setter
    def root(self, value: str) -> None:
        """Point the chain (and every block it knows) at a copy of the directory."""
        self._root = value
        for b in self.blocks:
            b.root = value

    def __repr__(self) -> str:
        cur = self.blocks[min(self.block_id, len(self.blocks) - 1)]
        return (f"Chain of {len(self.blocks)} known blocks:\n > root        = {self.root}\n > block id    = {self.block_id}\n"
                f" > block file  = {cur.target_path}\n > in-block id = {self.in_block_id}")

    # ------------------------------------------------------------------ the whole chain at once
    def extend(self) -> int:
        """Follow the links to the end and remember every block (without keeping their data); returns the number
        of blocks known afterwards.  A link to a file that is not there yet ends the walk."""
        with self._lock:
            while True:
                tail = self.blocks[-1]
                try:
                    was = tail.loaded
                    if not was:
                        tail.load()
                    nxt = list(tail.next)
                    if not was and len(self.blocks) > 1:
                        tail.unload()
                except OSError:
                    break
                if nxt[0] is None or not os.path.exists(os.path.join(self.root, nxt[0])):
                    break
                self.blocks.append(Block(self.root, nxt[0], nxt[1], verify=self.verify))
            return len(self.blocks)

    def fastload(self) -> int:
        """Index the data blocks from the directory listing (``block_<n>_*.pkl`` in order of ``n``) instead of
        walking the links, and switch checksum verification off: for chains of many blocks on a slow filesystem."""
        import re

        if len(self.blocks) != 1:
            raise AssertionError("fastload starts from a fresh chain")
        found = sorted((int(re.match(r"block_(\d+)_", f).group(1)), f) for f in self._all_files())
        self.verify = False
        first = found[0][0] if found else 1                   # chains written by early versions of this module start at 0
        for want, (idx, f) in enumerate(found, start=first):
            if idx != want:
                raise AssertionError(f"block {want} is missing from {self.root} (found block {idx})")
            self.blocks.append(Block(self.root, f, verify=False))
        return len(found)

    def validate(self) -> list:
        """Walk the chain and compare every block with the checksum its predecessor recorded.  Returns
        ``[(file, samples, ok)]``; nothing is kept in memory."""
        self.extend()
        out, expect = [], None
        for blk in self.blocks:
            held = blk.loaded
            if not held:
                with open(blk.target_path, "rb") as f:
                    data, nxt = pickle.load(f)
            else:
                data, nxt = blk.data, blk.next
            ok = expect in (None, "", "EMPTY") or md5(pickle.dumps(data)).hexdigest() == expect
            out.append((blk.target_file, len(data), ok))
            expect = nxt[1] if nxt and nxt[0] is not None else None
        return out

    # ------------------------------------------------------------------ writing
    @contextlib.contextmanager
    def writer(self, block_size: int = 1000):
        """``with chain.writer(1000) as write: write(sample)`` appends after the current last block."""
        last = self._walk_to_end()
        buf: list = []
        # data blocks are numbered from 1 (the root block is number 0), as the reference's writer numbers them and
        # its ``fastload`` expects
        used = [int(f.split("_")[1]) for f in self._all_files()]
        index = [max(used) + 1 if used else 1]

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

    def run_loader(self) -> None:
        """Start the prefetch thread (``get`` does it on first use when ``prefetch`` > 0)."""
        if self.prefetch and self._loader is None:
            self._loader = threading.Thread(target=self._prefetch_loop, daemon=True)
            self._loader.start()

    def _seek_sample(self) -> Block | None:
        """Move the position onto the next existing sample (skipping exhausted and empty blocks, wrapping to the
        first block once); returns its block, or None for a chain without samples."""
        self.run_loader()
        for _ in range(2):
            blk = self._block(self.block_id)
            while blk is not None and self.in_block_id >= len(blk):
                if self.block_id > 1 and not self.reusable:
                    with self._lock:
                        self.blocks[self.block_id - 1].unload()
                self.block_id, self.in_block_id = self.block_id + 1, 0
                blk = self._block(self.block_id)
            if blk is not None:
                return blk
            if len(self.blocks) <= 1:
                return None
            logger.warning(f"{len(self.blocks)=}. next_block is empty, restart from root!!!")
            self.block_id, self.in_block_id = 0, 0
        return None

    def get_nostep(self):
        """The sample ``get`` would return, without consuming it."""
        blk = self._seek_sample()
        return None if blk is None else blk.data[self.in_block_id]

    def next(self) -> bool:
        """Consume one sample without reading it; False for a chain without samples."""
        if self._seek_sample() is None:
            return False
        self.in_block_id += 1
        return True

    def get(self):
        """Next sample; after the last block the chain restarts from the first one. ``None`` for an empty chain."""
        blk = self._seek_sample()
        if blk is None:
            return None
        item = blk.data[self.in_block_id]
        self.in_block_id += 1
        return item

    def __iter__(self):
        return self

    def __next__(self):
        item = self.get()
        if item is None:
            raise StopIteration
        return item

    def state_dict(self) -> dict:
        return {"root": self.root, "blocks": [b.state_dict() for b in self.blocks], "block_id": self.block_id,
                "in_block_id": self.in_block_id}

    def load_state_dict(self, state: dict) -> None:
        """Position, and - when the state carries them - root and block list (a state saved by the reference does)."""
        if state.get("root"):
            self.root = state["root"]
        if state.get("blocks"):
            with self._lock:
                self.blocks = [Block(self.root, b["target_file"], b.get("checksum", "EMPTY"), b.get("next"), verify=self.verify)
                               for b in state["blocks"]]
        self.block_id, self.in_block_id = state["block_id"], state["in_block_id"]

    def close(self) -> None:
        self._stop = True
