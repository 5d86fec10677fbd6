"""Indexed binary shards: slice arithmetic against Python's own slicing, raw / pickled / typed records, per-item reads."""
import itertools
import os
import pickle

import numpy as np
import pytest

from steptronoss_b200.data.indexed_bin import (AutoReader, FileReader, IndexedBinReader, IndexedBinWriter, compute_span,
                                               normalize_slice, pread, readexactly)


def test_slice_arithmetic_matches_python_slicing():
    values = [None, -7, -3, -1, 0, 1, 2, 4, 5, 9]
    for size in (0, 1, 5):
        x = list(range(size))
        for start, stop, step in itertools.product(values, values, [None, 1, 2, 3, -1, -2]):
            want = x[slice(start, stop, step)]
            a, b, c = normalize_slice(size, start, stop, step)
            got, i = [], a
            while i != b:
                assert 0 <= i < size
                got.append(x[i])
                i += c
            assert got == want, (size, start, stop, step)
            lo, hi = compute_span(size, start, stop, step)
            assert x[lo:hi][::step] == want and (lo == hi or (0 <= lo < size and 0 < hi <= size))
    with pytest.raises(ValueError):
        normalize_slice(4, None, None, 0)


def test_typed_shard_reads_items_and_slices_without_the_rest(tmp_path):
    docs = [np.arange(10, dtype=np.int32), np.arange(100, 103, dtype=np.int32), np.zeros(0, dtype=np.int32)]
    with IndexedBinWriter(str(tmp_path), prefix="tok_", cfg={"dtype": "int32"}) as w:
        sizes = [w.write(d.tobytes()) for d in docs]
        assert sizes == [40, 12, 0] and w.tell() == 52
    assert sorted(os.listdir(tmp_path)) == [".success", "cfg.json", "tok_data.bin", "tok_index.npz"]
    r = IndexedBinReader(str(tmp_path), prefix="tok_")
    assert len(r) == 3 and r.dtype == np.int32 and list(r.sizes) == [10, 3, 0] and list(r.offsets) == [0, 10, 13]
    assert np.array_equal(r[0], docs[0]) and np.array_equal(r[1, ...], docs[1]) and r[2].size == 0
    assert r[0, 3] == 3 and r[1, -1] == 102
    assert np.array_equal(r[0, 2:9:3], docs[0][2:9:3]) and np.array_equal(r[0, ::-2], docs[0][::-2])
    with pytest.raises(IndexError):
        r[1, 3]
    again = pickle.loads(pickle.dumps(r))                       # what a dataloader worker receives
    assert np.array_equal(again[0, 5:], docs[0][5:]) and again.read_bytes(1) == docs[1].tobytes()
    r.close()


def test_pickled_records_raw_bytes_and_aborted_writers(tmp_path):
    good, bad = tmp_path / "good", tmp_path / "bad"
    with IndexedBinWriter(str(good)) as w:
        assert w.append({"tokens": [1, 2, 3]}) == 0 and w.append("text") == 1
        w.write(b"raw!")
    r = IndexedBinReader(str(good))
    assert r[0] == {"tokens": [1, 2, 3]} and r[1] == "text" and r.read_bytes(2) == b"raw!" and r[2, 1:3] == b"aw"
    with pytest.raises(RuntimeError):
        with IndexedBinWriter(str(bad)) as w:
            w.write(b"half a shard")
            raise RuntimeError("producer failed")
    assert not os.path.exists(bad / ".success")
    with pytest.raises(FileNotFoundError):
        IndexedBinReader(str(bad))
    # byte sources
    f = FileReader(str(good / "data.bin"))
    assert isinstance(AutoReader(str(good / "data.bin")), FileReader) and bytes(f.read(r.offsets[2], 4)) == b"raw!"
    with open(good / "data.bin", "rb", buffering=0) as fh:
        head = readexactly(fh, 5)
        assert bytes(pread(fh, 0, 5)) == head and fh.tell() == 5         # pread leaves the position alone
        with pytest.raises(OSError):
            pread(fh, 0, 10 ** 6)
    with pytest.raises(RuntimeError, match="s3://"):
        AutoReader("s3://bucket/shard/data.bin")
