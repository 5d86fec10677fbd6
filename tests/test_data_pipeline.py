"""Data pipeline: packing, samplers, DP multiplexing and state round trips."""
from steptronoss_b200.data.nextable import DPMux
from steptronoss_b200.data.packing import pack
from steptronoss_b200.data.samplers import LoopedSequentialSampler, LoopedShuffleSampler, WeightedRandomSampler


def test_pack_greedy_exact_fit_drop_and_extend():
    r = pack([3, 4, 5, 2, 12, 1, 9], 10, "drop")
    assert r.packed_sample_ranges == [(0, 2), (2, 2), (5, 2)] and r.num_droped == 1
    r = pack([3, 4, 5, 2, 12, 1, 9], 10, "extend")
    assert r.packed_sample_ranges == [(0, 2), (2, 2), (4, 1), (5, 2)] and r.num_droped == 0
    assert pack([5, 5, 5], 10).packed_sample_ranges == [(0, 2), (2, 1)]
    assert pack([], 10).num_packed_samples == 0


def test_samplers_loop_and_resume():
    s = LoopedSequentialSampler(3)
    assert [next(s) for _ in range(7)] == [0, 1, 2, 0, 1, 2, 0]
    sh = LoopedShuffleSampler(5, seed=1)
    first = [next(sh) for _ in range(10)]
    assert sorted(first[:5]) == list(range(5)) and sorted(first[5:]) == list(range(5)) and first[:5] != first[5:]
    st = sh.state_dict()
    nxt = [next(sh) for _ in range(4)]
    sh2 = LoopedShuffleSampler(5, seed=1)
    sh2.load_state_dict(st)
    assert [next(sh2) for _ in range(4)] == nxt


def test_weighted_sampler_follows_weights():
    w = WeightedRandomSampler([1, 3])
    picks = [next(w) for _ in range(400)]
    assert abs(picks.count(1) - 300) <= 1


def test_dpmux_partitions_stream_and_resumes():
    streams = [DPMux(LoopedSequentialSampler(100), 3, r) for r in range(3)]
    got = [[next(s) for _ in range(4)] for s in streams]
    assert got == [[0, 3, 6, 9], [1, 4, 7, 10], [2, 5, 8, 11]]
    state = streams[0].state_dict()
    resumed = [DPMux(LoopedSequentialSampler(100), 3, r) for r in range(3)]
    for s in resumed:
        s.load_state_dict(state)
    assert [next(s) for s in resumed] == [12, 13, 14]


# ---------------------------------------------------------------------------- loaders, recipe, async workers
class _ToyDs:
    def __init__(self, n, base, lens):
        self.items = [{"tokens": [base + i] * lens[i % len(lens)]} for i in range(n)]
        self.sample_meta = [len(x["tokens"]) for x in self.items]

    def __len__(self):
        return len(self.items)

    def __getitem__(self, i):
        return self.items[i]


def test_mixed_packed_dataloader_mixture_packing_and_resume():
    from steptronoss_b200.data.dataloader import MixedPackedDataloader

    a, b = _ToyDs(20, 0, [3, 5, 7]), _ToyDs(10, 1000, [4, 6])
    dl = MixedPackedDataloader([a, b], [1.0, 2.0], max_length=16, dataset_sampling=["sequential", "random"])
    seen = [next(dl) for _ in range(len(dl))]
    flat = [x["tokens"][0] for pack_ in seen for x in pack_]
    assert sum(1 for t in flat if t < 1000) == 20 and sum(1 for t in flat if t >= 1000) == 20   # 1 and 2 epochs
    assert all(sum(len(x["tokens"]) for x in p) <= 16 for p in seen)
    assert [t for t in flat if t < 1000] == list(range(20))                                       # sequential domain
    dl2 = MixedPackedDataloader([a, b], [1.0, 2.0], max_length=16, dataset_sampling=["sequential", "random"])
    for _ in range(3):
        next(dl2)
    st = dl2.state_dict()
    dl3 = MixedPackedDataloader([a, b], [1.0, 2.0], max_length=16, dataset_sampling=["sequential", "random"])
    dl3.load_state_dict(st)
    assert next(dl3) == seen[3]


def test_recipe_validation():
    import pytest as _pt

    from steptronoss_b200.data.recipe import CompiledDataRecipe, DataRecipe, DataSourceFile

    r = DataRecipe({"a": [DataSourceFile("x.jsonl", 0.5)]}, {"a": 2.0})
    assert r == DataRecipe({"a": [DataSourceFile("x.jsonl", 0.5)]}, {"a": 2.0}) and r.to_dict()["epochs"] == {"a": 2.0}
    with _pt.raises(ValueError):
        DataSourceFile("x", 0.0)
    with _pt.raises(ValueError):
        DataRecipe({"a": []}, {"b": 1.0})
    with _pt.raises(ValueError):
        DataRecipe({"a": [], "b": []}, {"a": 1.0})
    with _pt.raises(ValueError):
        CompiledDataRecipe({"a": "/p"}, {"a": 0.0})


class _Counter:
    """SlowFastNextable over the integers with a visible cost for building an item."""

    def __init__(self):
        self.i = 0

    def __iter__(self):
        return self

    def __next__(self):
        import torch as _t

        v = self.i
        self.i += 1
        return {"x": _t.full((4,), v)}

    def fast_step(self):
        self.i += 1

    def state_dict(self):
        return {"i": self.i}

    def load_state_dict(self, s):
        self.i = s["i"]


def test_async_accelerated_stream_is_the_serial_stream_and_resumes():
    from steptronoss_b200.data.async_accelerate import AsyncAcceleratedSlowFast
    from steptronoss_b200.data.nextable import SlowFastNextable

    SlowFastNextable.register(_Counter)
    acc = AsyncAcceleratedSlowFast(_Counter(), queue_size=12, num_workers=3)
    try:
        got = [int(next(acc)["x"][0]) for _ in range(10)]
        assert got == list(range(10))
        st = acc.state_dict()
        assert st == {"i": 10}
        acc.load_state_dict({"i": 4})
        assert [int(next(acc)["x"][0]) for _ in range(5)] == [4, 5, 6, 7, 8]
    finally:
        acc.close()
