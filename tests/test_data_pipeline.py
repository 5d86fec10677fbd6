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


def test_sft_pack_contract_and_training_on_packed_chat_samples():
    import torch

    from steptronoss_b200.exp.lr_schedulers import ConstantSchedulerConfig
    from steptronoss_b200.exp.sft import SFTDataConfig, SFTDatasetsConfig, SFTExp

    class Chat:
        """prompt tokens masked out, answer = prompt reversed (learnable)"""

        def __init__(self, n, seed):
            import random as _r

            rnd = _r.Random(seed)
            self.items = []
            for _ in range(n):
                p = [rnd.randrange(2, 30) for _ in range(rnd.randint(3, 8))]
                toks = [1] + p + [31] + p[::-1] + [0]
                mask = [0] * (len(p) + 2) + [1] * (len(p) + 1)
                self.items.append({"tokens": toks, "loss_mask": mask})
            self.sample_meta = [len(x["tokens"]) for x in self.items]

        def __len__(self):
            return len(self.items)

        def __getitem__(self, i):
            return self.items[i]

    class Sets(SFTDatasetsConfig):
        def build_datasets(self):
            return {"a": (Chat(40, 0), 1.0), "b": (Chat(20, 1), 2.0)}

    class Data(SFTDataConfig):
        dataset_cfg = Sets
        num_workers = 0

    class Exp(SFTExp):
        data_cfg = Data
        scheduler_cfg = ConstantSchedulerConfig

    e = Exp()
    m = e.model_cfg
    m.num_layers, m.hidden_size, m.params_dtype, m.variable_seq_lengths = 2, 32, torch.float32, True
    a = m.attn_cfg
    a.num_attention_heads, a.num_attention_groups, a.head_dim, a.hidden_size = 2, 1, 16, 32
    m.ffn_cfg.hidden_size, m.ffn_cfg.ffn_hidden_size = 32, 64
    m.tok_embed_cfg.vocab_size = m.out_embed_cfg.vocab_size = 32
    m.tok_embed_cfg.hidden_size = m.out_embed_cfg.hidden_size = 32
    m.parallel_cfg.expert_tensor_parallel_size = 1
    t = e.trainer_cfg
    t.global_batch_size, t.global_seq_length, t.train_iters, t.writer_backend = 2, 64, 8, []
    e.scheduler_cfg.lr, e.scheduler_cfg.weight_decay, e.scheduler_cfg.warmup_schedule = 3e-3, 0.0, 0
    e.data_cfg.seqlen_divisible_by = 8

    dl = e.data_cfg.build_dataloader(0, 1)
    batch = next(dl)
    n = batch["tokens"].numel()
    assert n % 8 == 0 and n <= 64 and batch["cu_seqlens"].dtype == torch.int32 and int(batch["cu_seqlens"][-1]) == n
    first_doc = slice(0, int(batch["cu_seqlens"][1]))
    assert torch.equal(batch["labels"][first_doc][:-1], batch["tokens"][first_doc][1:])   # shift by one inside a doc
    assert batch["position_id"][first_doc].tolist() == list(range(first_doc.stop))
    assert float(batch["loss_mask"][int(batch["cu_seqlens"][-2]):].sum()) >= 0            # padding doc is masked out

    tr = e.trainer_cfg.get_trainer_cls()(exp=e)
    tr.before_train()
    losses = []
    for _ in range(8):
        tr.train_step()
        tr.iteration += 1
        tr.training_log()
        losses.append(tr.history[-1]["lm_loss"])
    assert losses[-1] < losses[0]


def test_blockchain_write_copy_read_resume(tmp_path):
    import shutil

    from steptronoss_b200.data.blockchain import Chain

    src = tmp_path / "a"
    chain = Chain(str(src))
    with chain.writer(block_size=4) as write:
        for i in range(10):
            write({"i": i})
    with Chain(str(src)).writer(block_size=4) as write:       # append later
        write({"i": 10})
    dst = tmp_path / "b"
    shutil.copytree(src, dst)
    rd = Chain(str(dst), prefetch=1)
    got = [rd.get()["i"] for _ in range(11)]
    assert got == list(range(11))
    assert rd.get()["i"] == 0                                   # wraps around like a training stream
    rd2 = Chain(str(dst))
    for _ in range(6):
        rd2.get()
    st = rd2.state_dict()
    rd3 = Chain(str(dst))
    rd3.load_state_dict(st)
    assert rd3.get()["i"] == 6
    rd.close()
    # peek / skip, the whole chain at once, a moved directory
    walk = Chain(str(dst), reusable=True)
    assert walk.get_nostep()["i"] == 0 and walk.get_nostep()["i"] == 0 and walk.next() and walk.get()["i"] == 1
    assert walk.extend() == 5                                   # root + 3 blocks of the first writer + 1 appended
    assert [(n, ok) for _, n, ok in walk.validate()] == [(0, True), (4, True), (4, True), (2, True), (1, True)]
    assert all(b.loaded for b in walk.blocks[:2])               # reusable: what was read stays in memory
    quick = Chain(str(dst))
    assert quick.fastload() == 4 and not quick.verify and [quick.get()["i"] for _ in range(11)] == list(range(11))
    moved = tmp_path / "c"
    shutil.move(str(dst), str(moved))
    walk.root = str(moved)
    assert walk.get()["i"] == 2 and str(moved) in repr(walk) and "in-block id" in repr(walk)
    other = Chain(str(tmp_path / "elsewhere"))
    other.load_state_dict(walk.state_dict())                    # a full state carries root and blocks along
    assert other.root == str(moved) and other.get()["i"] == 3
    blk = walk.blocks[2]
    blk.load()
    blk.data[0] = {"i": -1}
    blk.save()                                                  # a block changed behind the chain's back
    assert [ok for _, _, ok in Chain(str(moved)).validate()] == [True, True, False, True, True]
    empty = Chain(str(tmp_path / "nothing"))
    assert empty.get() is None and empty.get_nostep() is None and not empty.next()


def test_samplers_cover_epochs_resume_and_skip_without_building_items():
    from steptronoss_b200.data.nextable import DPMux, Nextable, SlowFastNextable
    from steptronoss_b200.data.samplers import LoopedSequentialSampler, LoopedShuffleSampler

    seq = LoopedSequentialSampler(3)
    assert [next(seq) for _ in range(7)] == [0, 1, 2, 0, 1, 2, 0] and isinstance(seq, Nextable)
    sh = LoopedShuffleSampler(5, seed=3)
    first, second = [next(sh) for _ in range(5)], [next(sh) for _ in range(5)]
    assert sorted(first) == sorted(second) == [0, 1, 2, 3, 4] and first != second      # a new order every epoch
    again = LoopedShuffleSampler(5, seed=3)
    for _ in range(3):
        again.fast_step()                                                              # skipping == taking
    assert [next(again) for _ in range(2)] == first[3:]
    state = again.state_dict()
    resumed = LoopedShuffleSampler(5, seed=99)
    resumed.load_state_dict(state)                                                     # the seed travels with the state
    assert [next(resumed) for _ in range(5)] == second

    class Plain:                                                                       # duck-typed protocol member
        def __next__(self):
            return 1

        def state_dict(self):
            return {}

        def load_state_dict(self, sd):
            pass

    assert isinstance(Plain(), Nextable) and not isinstance(Plain(), SlowFastNextable)
    ranks = [DPMux(LoopedSequentialSampler(100), dp_size=3, dp_rank=r) for r in range(3)]
    taken = [[next(m) for _ in range(3)] for m in ranks]
    assert taken == [[0, 3, 6], [1, 4, 7], [2, 5, 8]]


def test_local_futures_and_get_ready():
    import threading
    import time

    import pytest

    from steptronoss_b200.utils.comm_utils import LocalFuture, get_ready, wait_by_finish_order

    a, b, c = LocalFuture(), LocalFuture(), LocalFuture()
    assert not a.completed
    with pytest.raises(TimeoutError):
        a.result(timeout=0.05)
    ready, pending = get_ready([a, b], timeout=0.05)
    assert ready == [] and pending == [a, b]
    b.set_result("b")
    ready, pending = get_ready([a, b, c])
    assert ready == [b] and pending == [a, c] and b.result() == "b"
    with pytest.raises(AssertionError):
        b.set_result("again")
    threading.Thread(target=lambda: (time.sleep(0.1), c.set_result(3), time.sleep(0.1), a.set_result(None))).start()
    order = [f for f in wait_by_finish_order([a, c])]
    assert order == [c, a] and a.completed and a.result() is None                      # None is a value, not "pending"


def _ignores_sigterm():
    import signal
    import time

    signal.signal(signal.SIGTERM, signal.SIG_IGN)
    time.sleep(60)


def test_soft_kill_ends_a_worker_that_ignores_the_polite_request():
    import multiprocessing as mp
    import time

    from steptronoss_b200.data.async_accelerate import soft_kill_process

    p = mp.get_context("fork").Process(target=_ignores_sigterm)
    p.start()
    time.sleep(0.3)
    t0 = time.time()
    soft_kill_process(p, timeout=0.5)
    assert not p.is_alive() and time.time() - t0 < 5
