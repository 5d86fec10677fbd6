"""Indexed binary shards (reference ``steptronoss/data/utils/indexed_bin_file.py:11-366``).

A shard directory holds ``<prefix>data.bin`` (the records back to back), ``<prefix>index.npz`` (``offsets`` and
``sizes`` in bytes, little-endian uint64), an optional ``cfg.json`` (``{"dtype": ...}`` makes the records typed arrays)
and a ``.success`` marker written last.  A record is raw bytes (``write``), a pickled object (``append``) or, with a
dtype, an array of items; typed shards are addressed per item: ``reader[i, j]`` is one item of record ``i`` and
``reader[i, a:b:c]`` a strided slice, read without touching the rest of the record.  Readers use ``os.pread`` on a
descriptor opened at first use, so forked workers and unpickled copies do not share a file position.
"""
from __future__ import annotations

import json
import os
import pickle

import numpy as np


# ---- slices --------------------------------------------------------------------------------------------------------
def normalize_slice(size: int, start, stop, step):
    """``(start, stop, step)`` with every ``None`` and negative index resolved against ``size``, clipped, and ``stop``
    moved onto the stride, so that ``i = start; while i != stop: use x[i]; i += step`` visits exactly
    ``x[start:stop:step]`` and every ``i`` is a valid index."""
    step = 1 if step is None else step
    if step == 0:
        raise ValueError("slice step cannot be zero")
    lo, hi = (0, size) if step > 0 else (-1, size - 1)            # clip range of both ends for this direction
    first_default, stop_default = (0, size) if step > 0 else (size - 1, -1)
    start = first_default if start is None else (start + size if start < 0 else start)
    stop = stop_default if stop is None else (stop + size if stop < 0 else stop)
    start, stop = min(max(start, lo), hi), min(max(stop, lo), hi)
    count = max((stop - start + (-1 if step > 0 else 1)) // step + 1, 0)
    return start, start + count * step, step


def compute_span(size: int, start, stop, step):
    """The contiguous ``[lo, hi)`` that contains ``x[start:stop:step]``: ``x[lo:hi][::step]`` is that slice (for a
    negative step the span is read forwards and reversed by the stride)."""
    start, stop, step = normalize_slice(size, start, stop, step)
    count = (stop - start) // step
    if count == 0:
        return start, start
    last = start + step * (count - 1)
    return (start, last + 1) if step > 0 else (last, start + 1)


# ---- byte sources --------------------------------------------------------------------------------------------------
def readexactly(file, size: int) -> bytes:
    """``size`` bytes from the current position of an unbuffered file, however the reads are split up."""
    buf = memoryview(bytearray(size))
    got = 0
    while got < size:
        n = file.readinto(buf[got:])
        if not n:
            raise OSError(f"{getattr(file, 'name', file)}: file ended after {got} of {size} bytes")
        got += n
    return bytes(buf)


def pread(file, offset: int, size: int) -> bytearray:
    """``size`` bytes at ``offset`` without moving the file position (safe across forked workers)."""
    out = bytearray(size)
    got = 0
    while got < size:
        chunk = os.pread(file.fileno(), size - got, offset + got)
        if not chunk:
            raise OSError(f"{file.name}: file ended {size - got} bytes short of a record")
        out[got:got + len(chunk)] = chunk
        got += len(chunk)
    return out


class FileReader:
    """Positional reads from a local file, opened at first use; pickles as the path alone."""

    def __init__(self, path: str) -> None:
        self.path = path
        self.file = None

    def read(self, offset: int, size: int) -> bytearray:
        if self.file is None:
            self.file = open(self.path, "rb", buffering=0)
        return pread(self.file, int(offset), int(size))

    def close(self) -> None:
        if self.file is not None:
            self.file.close()
            self.file = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def __getstate__(self):
        return {"path": self.path}

    def __setstate__(self, state):
        self.path, self.file = state["path"], None


class S3Reader:
    """Ranged GETs from an object store.  The client library is not part of this image, so construction says so;
    the class exists so that ``AutoReader`` fails with a clear message instead of a missing name."""

    def __init__(self, path: str) -> None:
        raise RuntimeError(f"{path}: reading shards from s3:// needs boto3 / megfile, which are not installed; "
                           "copy the shard to a local or mounted path")


def AutoReader(path: str):  # noqa: N802  (the reference's name)
    return S3Reader(path) if path.startswith("s3://") else FileReader(path)


# ---- writer --------------------------------------------------------------------------------------------------------
class IndexedBinWriter:
    def __init__(self, path: str, prefix: str = "", cfg: dict | None = None):
        self.path, self.prefix = path, prefix
        os.makedirs(path, exist_ok=True)
        self._f = open(os.path.join(path, prefix + "data.bin"), "wb")
        self._offsets, self._sizes, self._pos = [], [], 0
        self._cfg = cfg

    def write(self, data) -> int:
        """Append one record of raw bytes (anything with the buffer protocol); returns its size."""
        if self._f is None:
            raise ValueError("writer is closed")
        view = memoryview(data).cast("B")
        self._f.write(view)
        self._offsets.append(self._pos)
        self._sizes.append(view.nbytes)
        self._pos += view.nbytes
        return view.nbytes

    def append(self, record) -> int:
        """Append one pickled object; returns its index."""
        self.write(pickle.dumps(record, protocol=pickle.HIGHEST_PROTOCOL))
        return len(self._offsets) - 1

    def tell(self) -> int:
        return self._pos

    def close(self) -> None:
        if self._f is None:
            return
        self._f.close()
        self._f = None
        np.savez_compressed(os.path.join(self.path, self.prefix + "index.npz"),
                            offsets=np.asarray(self._offsets, dtype="<u8"), sizes=np.asarray(self._sizes, dtype="<u8"))
        if self._cfg:
            with open(os.path.join(self.path, "cfg.json"), "w") as f:
                json.dump(self._cfg, f)
        open(os.path.join(self.path, ".success"), "w").close()

    def abort(self) -> None:
        """Stop without an index and without ``.success``: readers refuse the directory."""
        if self._f is not None:
            self._f.close()
            self._f = None

    def __enter__(self):
        return self

    def __exit__(self, exc_type, exc, tb):
        if exc_type is None:
            self.close()
        else:
            self.abort()


# ---- reader --------------------------------------------------------------------------------------------------------
class IndexedBinReader:
    def __init__(self, path: str, dtype=None, prefix: str = ""):
        self.path, self.prefix = path, prefix
        self.dtype = None if dtype is None else np.dtype(dtype)
        cfg_file = os.path.join(path, "cfg.json")
        if os.path.exists(cfg_file):
            with open(cfg_file) as f:
                cfg = json.load(f)
            if "dtype" in cfg:
                self.dtype = np.dtype(cfg["dtype"])
        if not os.path.exists(os.path.join(path, ".success")):
            raise FileNotFoundError(f"{path} is not a complete indexed-bin shard (.success missing)")
        self.data_reader = AutoReader(os.path.join(path, prefix + "data.bin"))
        self._offsets = self._sizes = None

    @property
    def _itemsize(self) -> int:
        return 1 if self.dtype is None else self.dtype.itemsize

    def _load_index(self) -> None:
        idx = np.load(os.path.join(self.path, self.prefix + "index.npz"))
        self._offsets, r0 = np.divmod(idx["offsets"], self._itemsize)
        self._sizes, r1 = np.divmod(idx["sizes"], self._itemsize)
        if r0.any() or r1.any():
            raise ValueError(f"{self.path}: record boundaries are not multiples of the {self.dtype} item size")

    @property
    def offsets(self):
        """Start of every record, in items (bytes without a dtype)."""
        if self._offsets is None:
            self._load_index()
        return self._offsets

    @property
    def sizes(self):
        if self._sizes is None:
            self._load_index()
        return self._sizes

    def __getstate__(self):
        return {"path": self.path, "prefix": self.prefix, "dtype": self.dtype, "data_reader": self.data_reader}

    def __setstate__(self, state):
        self.__dict__.update(state)
        self._offsets = self._sizes = None

    def _read_span(self, i: int, start: int, stop: int):
        raw = self.data_reader.read((int(self.offsets[i]) + start) * self._itemsize, (stop - start) * self._itemsize)
        return raw if self.dtype is None else np.frombuffer(raw, dtype=self.dtype)

    def read_bytes(self, i: int) -> bytes:
        """Record ``i`` as stored."""
        n = int(self.sizes[i]) * self._itemsize
        return bytes(self.data_reader.read(int(self.offsets[i]) * self._itemsize, n))

    def __len__(self) -> int:
        return len(self.offsets)

    def __getitem__(self, arg):
        """``reader[i]``: the record - unpickled for untyped shards, an array for typed ones.  ``reader[i, j]``: item
        ``j`` of record ``i``; ``reader[i, a:b:c]`` or ``reader[i, ...]``: a slice of its items (typed shards; on an
        untyped shard the items are bytes)."""
        if not isinstance(arg, tuple):
            if self.dtype is None:
                return pickle.loads(self.read_bytes(arg))
            return self._read_span(arg, 0, int(self.sizes[arg]))
        i, j = (arg[0], Ellipsis) if len(arg) == 1 else arg
        size = int(self.sizes[i])
        if j is Ellipsis:
            return self._read_span(i, 0, size)
        if isinstance(j, slice):
            lo, hi = compute_span(size, j.start, j.stop, j.step)
            return self._read_span(i, lo, hi)[::j.step]
        j = j + size if j < 0 else j
        if not 0 <= j < size:
            raise IndexError(f"item {arg[1]} of a record with {size} items")
        return self._read_span(i, j, j + 1)[0]

    def close(self) -> None:
        if getattr(self, "data_reader", None) is not None:
            self.data_reader.close()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
