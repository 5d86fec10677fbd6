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
