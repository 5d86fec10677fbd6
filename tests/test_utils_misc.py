"""Small utilities: timers, memory marks, RNG streams with recompute, the step writer, CLI overrides."""
import os
import time

import pytest
import torch


def test_timers_levels_scopes_and_report():
    from steptronoss_b200.utils.timers import get_timers, init_timers, timeit

    t = init_timers(log_level=1, use_event=False)
    with t.record("coarse", 1):
        time.sleep(0.02)
    with t.record("fine", 2):          # above the log level: not recorded
        time.sleep(0.01)
    t("manual").start()
    time.sleep(0.01)
    t("manual").stop()

    @timeit("decorated", log_level=1)
    def f(x):
        time.sleep(0.01)
        return x + 1

    assert f(1) == 2 and get_timers() is t
    rep = t.report(reset=False)
    assert set(rep) == {"coarse", "manual", "decorated"} and rep["coarse"] >= 15.0
    assert t.report(normalizer=2.0, reset=True)["coarse"] == pytest.approx(rep["coarse"] / 2, rel=0.05)
    assert t.report()["coarse"] == 0.0 and t.log_string().startswith("time (ms) | ")
    init_timers()


def test_timers_write_log_and_reload():
    from steptronoss_b200.utils.timers import DummyTimers, LocalTimers, init_timers

    t = init_timers(log_level=1, use_event=False)
    assert isinstance(t, LocalTimers) and not isinstance(t, DummyTimers)
    with t.record("step", 1):
        time.sleep(0.02)
    t("never-ran", 1)

    class Writer:
        def __init__(self):
            self.rows = []

        def add_scalar(self, name, value, it):
            self.rows.append((name, value, it))

    w = Writer()
    wrote = t.write(w, 7, normalizer=2.0)
    assert list(wrote) == ["step"] and w.rows == [("Timers/step", wrote["step"], 7)] and 0.005 < wrote["step"] < 0.05
    text = t.log(7, prefix="iteration 7/100")
    assert text.startswith("iteration 7/100 | Activated Timers:") and "step....." in text and "never-ran" not in text
    assert t.log(8) == ""                                         # the log reset the timers
    with t.record("fine", 2):
        pass
    assert "fine" not in t.timers
    t.reload(5, False)                                            # levels are capped at 2
    assert t.log_level == 2
    with t.record("fine", 2):
        time.sleep(0.005)
    assert t.report()["fine"] > 0
    d = DummyTimers()
    with d.record("anything", 0):
        pass
    d("x").start()
    assert d.report() == {} and d("x").elapsed() == 0.0
    init_timers()


def test_memory_marks_only_when_enabled(monkeypatch):
    from steptronoss_b200.utils import memory_tracker
    from steptronoss_b200.utils.memory_tracker import MemoryTracker

    # the resident set of a long test process need not grow when memory is recycled: count what the test allocates
    held = [1 << 30]
    monkeypatch.setattr(memory_tracker, "_rss_bytes", lambda: held[0])

    off = MemoryTracker(enabled=False)
    assert off.mark("a") is None and off.marks == []
    on = MemoryTracker(enabled=True)
    on.mark("start")
    blob = bytearray(64 << 20)
    held[0] += len(blob)
    m = on.mark("after-alloc")
    assert m.rss > 0 and len(on.marks) == 2
    name, d_gpu, d_rss = on.deltas()[0]
    assert name == "start -> after-alloc" and d_rss > 32 << 20 and d_gpu == 0
    rep = on.report()
    assert "after-alloc" in rep and "largest deltas" in rep
    del blob
    unnamed = on.mark()                                          # named after the calling module and line
    assert unnamed.name.startswith(__name__ + ":")
    rec = on.records()[-1]
    assert rec["mark"] == unnamed.name and rec["cpu_rss"] == float(held[0]) and rec["time"] > 0
    assert "largest peaks" in on.report_over_world()             # one process: this rank's report
    assert memory_tracker.get_caller_name() == __name__ and memory_tracker.get_caller_name(50) == "<unknown>"
    assert memory_tracker.CudaMemoryTracker is MemoryTracker
    on.reset()
    assert on.marks == []


def test_rng_tracker_streams_and_recompute_replays_dropout():
    from steptronoss_b200.parallel.random import checkpoint, get_rng_tracker

    tr = get_rng_tracker()
    tr.reset()
    torch.manual_seed(1)
    tr.add("model-parallel-rng", 1234)
    with pytest.raises(RuntimeError):
        tr.add("other", 1234)           # same seed twice
    with pytest.raises(RuntimeError):
        tr.add("model-parallel-rng", 99)
    before = torch.get_rng_state().clone()
    with tr.fork():
        a = torch.rand(4)
    assert torch.equal(torch.get_rng_state(), before)       # the default stream did not move
    with tr.fork():
        b = torch.rand(4)
    assert not torch.equal(a, b)                            # the named stream did
    saved = tr.get_states()
    with tr.fork():
        c = torch.rand(4)
    tr.set_states(saved)
    with tr.fork():
        assert torch.equal(torch.rand(4), c)

    def block(x):
        with tr.fork():
            return torch.nn.functional.dropout(x, 0.5, training=True) * 2

    x = torch.randn(64, requires_grad=True)
    states = tr.get_states()
    y = checkpoint(block, x)
    y.sum().backward()                                       # recompute must draw the same mask
    tr.set_states(states)
    x2 = x.detach().clone().requires_grad_()
    y2 = block(x2)
    y2.sum().backward()
    assert torch.equal(y, y2) and torch.equal(x.grad, x2.grad)
    tr.reset()


def test_step_writer_writes_event_files(tmp_path):
    from steptronoss_b200.utils.logger import StepWriter

    w = StepWriter(str(tmp_path / "tb"), backend=("tensorboard",))
    for i in range(3):
        w.add_scalar("loss", 1.0 / (i + 1), i)
    w.add_text("note", "hello", 0)
    w.add_histogram("h", torch.randn(10), 0)
    w.flush()
    w.close()
    files = os.listdir(tmp_path / "tb")
    assert any(f.startswith("events.out.tfevents") for f in files) or w.writers == []
    none = StepWriter(str(tmp_path / "none"), backend=())
    none.add_scalar("x", 1.0, 0)                            # no writers: a no-op, not an error
    none.close()


def test_cli_overrides_use_literals_and_existing_keys_only():
    from steptronoss_b200.config import Config
    from steptronoss_b200.config.arguments import parse_args

    class Inner(Config):
        lr: float = 1e-3
        name: str = "a"
        dims: list = [1, 2]

    class Exp(Config):
        inner = Inner
        steps: int = 10

    e = Exp()
    changes = e.merge(parse_args(["steps=20", "inner.lr=3e-4", "inner.name=hello", "inner.dims=[4,5]"]), exists_only=True)
    assert e.steps == 20 and e.inner.lr == 3e-4 and e.inner.name == "hello" and e.inner.dims == [4, 5]
    assert {c[0] for c in changes} == {"steps", "inner.lr", "inner.name", "inner.dims"}
    with pytest.raises(Exception):
        e.merge(parse_args(["inner.nope=1"]), exists_only=True)


def test_generic_load_by_extension_and_mode(tmp_path):
    import json
    import pickle

    import numpy as np

    from steptronoss_b200.utils.general import load

    (tmp_path / "a.json").write_text(json.dumps({"x": 1}))
    (tmp_path / "a.jsonl").write_text('{"i": 0}\n\n{"i": 1}\n')
    (tmp_path / "a.yaml").write_text("k: [1, 2]\n")
    (tmp_path / "a.txt").write_text("hello")
    (tmp_path / "weird.bin").write_text(json.dumps([3]))
    pickle.dump({"p": 2}, open(tmp_path / "a.pkl", "wb"))
    torch.save({"t": torch.arange(3)}, tmp_path / "a.pt")
    np.save(tmp_path / "a.npy", np.arange(4))
    assert load(str(tmp_path / "a.json")) == {"x": 1}
    assert load(str(tmp_path / "a.jsonl")) == [{"i": 0}, {"i": 1}]
    assert load(str(tmp_path / "a.yaml")) == {"k": [1, 2]} and load(str(tmp_path / "a.txt")) == "hello"
    assert load(str(tmp_path / "a.pkl")) == {"p": 2} and load(str(tmp_path / "a.pt"))["t"].tolist() == [0, 1, 2]
    assert load(str(tmp_path / "a.npy")).tolist() == [0, 1, 2, 3]
    assert load(str(tmp_path / "weird.bin"), mode="json") == [3]
    with pytest.raises(ValueError):
        load(str(tmp_path / "weird.bin"))


def test_debug_attach_only_listens_on_the_chosen_ranks(monkeypatch):
    import sys
    import types

    import steptronoss_b200

    calls = []
    fake = types.SimpleNamespace(is_client_connected=lambda: False,
                                 listen=lambda addr, in_process_debug_adapter=False: calls.append(("listen", addr[1])),
                                 wait_for_client=lambda: calls.append(("wait",)), breakpoint=lambda: calls.append(("break",)))
    monkeypatch.setitem(sys.modules, "debugpy", fake)
    assert steptronoss_b200.debug(rank=[3, 5]) is None and calls == []          # this process is rank 0
    host, port = steptronoss_b200.debug(rank=[2, 0], stop=True)
    assert port == 5001 and calls == [("listen", 5001), ("wait",), ("break",)]
    calls.clear()
    assert steptronoss_b200.debug(any_rank=True, base_port=6000)[1] == 6000
    fake.is_client_connected = lambda: True
    assert steptronoss_b200.debug(rank=0) is None


def test_capture_trace_writes_forward_and_backward_traces(tmp_path):
    import json

    from steptronoss_b200.utils.dev_utils import capture_trace

    fw, bw = str(tmp_path / "fw.json"), str(tmp_path / "bw.json")

    class M(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.lin = torch.nn.Linear(8, 8)

        @capture_trace(at=1, fw_file=fw, bw_file=bw, warmup=1)
        def forward(self, x):
            return self.lin(x).relu()

    m = M()
    for i in range(4):
        m(torch.randn(4, 8)).sum().backward()
        done = os.path.exists(fw) and os.path.exists(bw)
        assert done == (i >= 2)                 # the window opens at call warmup + at (the third call)
    for f in (fw, bw):
        events = json.load(open(f))["traceEvents"]
        assert len(events) > 0
    assert any(e.get("name") == "FW" for e in json.load(open(fw))["traceEvents"])


def test_misc_helpers(tmp_path, capsys):
    from steptronoss_b200.utils import misc

    assert misc.format_layermap({0: {0: {0: {"recompute": False}, 1: {"recompute": False}, 2: {"recompute": True}}},
                                 1: {0: {3: {"recompute": True}}}}) == (
        "pp0/vp0: 0-1: {recompute=False}; 2: {recompute=True}\npp1/vp0: 3: {recompute=True}")
    assert misc.get_path_tree_repr(["a/b/c.pt", "a/b/d.pt", "a/e.txt", "f"]).splitlines() == [
        "|-- a", "|   |-- b", "|   |   |-- c.pt", "|   |   +-- d.pt", "|   +-- e.txt", "+-- f"]
    assert misc.get_path_tree_repr([]) == ""
    recs = [{"a": 1}, {"b": "ü"}]
    assert misc.safe_dump_jsonl(recs, str(tmp_path / "x.jsonl")) and misc.load_jsonl(str(tmp_path / "x.jsonl")) == recs
    assert misc.safe_dump_jsonl(recs, str(tmp_path / "no" / "dir.jsonl")) is False            # logged, not raised
    assert misc.safe_dump_msgpack({"k": [1, 2, b"x"]}, str(tmp_path / "x.mp")) and misc.load_msgpack(str(tmp_path / "x.mp")) == {"k": [1, 2, b"x"]}
    (tmp_path / "src").mkdir()
    misc.check_and_link(str(tmp_path / "src"), str(tmp_path / "ln"))
    misc.check_and_link(str(tmp_path / "src") + "/", str(tmp_path / "ln"))                       # same target: fine
    with pytest.raises(OSError):
        misc.check_and_link(str(tmp_path / "other"), str(tmp_path / "ln"))
    d = misc.RepeatedDict()
    d["k"] = 1
    d["k"] = 2
    d.update({"k": 3, "j": 9}, repeat=2)
    assert len(d) == 6 and d["k"] == 1 and d.pop("k") == 1 and d.pop("k") == 2 and d.pop("missing") is None
    assert [d.pop("j"), d.pop("j"), d.pop("j")] == [9, 9, None] and "j" not in d
    d2 = misc.RepeatedDict()
    d2.load_state_dict(d.state_dict())
    assert len(d2) == 2 and d2["k"] == 3
    items = [{"t": torch.ones(2)}, {"t": torch.zeros(2)}]
    seen = [x["t"].sum().item() for x in misc.moving_iter(items, active="cpu", default="cpu")]
    assert seen == [2.0, 0.0]
    assert misc.cos_sim(torch.tensor([1.0, 0.0]), torch.tensor([2.0, 0.0])) == pytest.approx(1.0)
    assert "MemReport" in misc.get_mem_brief("x")
    misc.force_clear_mem()
    lin = torch.nn.Linear(3, 2, bias=False)
    with torch.no_grad():
        lin.weight.fill_(2.0)
    assert misc.calc_params_l2_norm([lin, lin]) == pytest.approx((6 * 4.0) ** 0.5)              # shared parameters once
    calls = []

    @misc.deprecated("use g")
    def f(x):
        calls.append(x)
        return x

    assert f(1) == 1 and f(2) == 2 and calls == [1, 2]
    bar = misc.GroupedProgressBar({"a": 2, "b": 1})
    bar.update("a")
    bar.update("b")
    assert bar.total_bar.n == 2 and bar.group_bars["a"].n == 1
    bar.close()


def test_patch_manager_replaces_wraps_and_restores():
    import json as json_mod

    import steptronoss_b200.utils.general as general
    from steptronoss_b200.utils.patch_utils import PatchesManager, get_func_name

    orig = general.safediv
    assert get_func_name(orig) == "steptronoss_b200.utils.general.safediv"
    PatchesManager.remove_patches()
    PatchesManager.register_patch("steptronoss_b200.utils.general.safediv", lambda n, d: -1)

    def doubling_wrapper(fn):
        return lambda *a, **k: 2 * fn(*a, **k)

    PatchesManager.register_patch(orig, doubling_wrapper)                                   # by function object
    with pytest.raises(RuntimeError):
        PatchesManager.register_patch("steptronoss_b200.utils.general.safediv", lambda n, d: 0)
    PatchesManager.register_patch("no.such.package.fn", None, create_dummy=True)
    PatchesManager.register_patch("json.brand_new_function", lambda: "new", create_dummy=True)
    PatchesManager.apply_patches()
    try:
        assert general.safediv(6, 3) == -2
        import importlib

        assert json_mod.brand_new_function() == "new"
        with pytest.raises(RuntimeError, match="does not exist"):
            importlib.import_module("no.such.package").fn()
    finally:
        PatchesManager.remove_patches()
    assert general.safediv is orig and general.safediv(6, 3) == 2 and not hasattr(json_mod, "brand_new_function")
    with pytest.raises((ModuleNotFoundError, AttributeError)):
        PatchesManager.register_patch("definitely.not.there.fn", lambda: 0).apply()
    PatchesManager.remove_patches()


def test_param_groups_by_multipliers_and_tags():
    from steptronoss_b200.optim.utils import advanced_get_param_groups

    m = torch.nn.Sequential(torch.nn.Linear(4, 4), torch.nn.LayerNorm(4), torch.nn.Linear(4, 2, bias=False))
    m[2].weight._lr_scale = 0.1
    m[0].weight.requires_grad_(False)
    groups = advanced_get_param_groups(m, is_matrix=lambda n, p: p.dim() == 2)
    keyed = {(g["wd_mult"], g["lr_mult"], g["is_matrix"]): len(g["params"]) for g in groups}
    assert keyed == {(0.0, 1.0, False): 3, (1.0, 0.1, True): 1}      # bias + two norm vectors; the scaled head; frozen weight left out
    opt = torch.optim.AdamW([{**g, "weight_decay": 0.1 * g["wd_mult"], "lr": 1e-3 * g["lr_mult"]} for g in groups])
    assert len(opt.param_groups) == 2


def test_tb_record_reads_back_what_the_step_writer_wrote(tmp_path):
    from steptronoss_b200.utils.dev_utils import TBRecord, text_chart
    from steptronoss_b200.utils.logger import StepWriter

    w = StepWriter(str(tmp_path / "run"))
    for i, v in enumerate([4.0, 2.0, 1.0, 0.5]):
        w.add_scalar("train/loss", v, i)
    w.flush()
    w.close()
    rec = TBRecord(str(tmp_path / "run"))
    assert "train/loss" in rec and "nope" not in rec and list(rec.keys()) == ["train/loss"]
    ev = rec["train/loss"]
    assert [e.step for e in ev] == [0, 1, 2, 3] and rec.values("train/loss") == [4.0, 2.0, 1.0, 0.5]
    chart = rec.asciichart("train/loss", height=4)
    lines = chart.split("\n")
    assert len(lines) == 4 and lines[0].lstrip().startswith("4.000e+00") and lines[-1].lstrip().startswith("5.000e-01")
    assert lines[0].split("|", 1)[1][0] == "*" and lines[-1].rstrip().endswith("*") and repr(chart) == str(chart)
    long = text_chart(range(1000), height=5, width=50)
    assert all(len(line.split("|", 1)[1]) == 50 for line in long.split("\n"))
    assert text_chart([]) == "(no values)" and "*" in text_chart([1.0, 1.0])


def test_timeit_takes_the_function_name_and_the_level_alias():
    import time

    import pytest

    from steptronoss_b200.utils.timers import init_timers, timeit

    timers = init_timers(log_level=1, use_event=False)

    @timeit()
    def plain_work():
        time.sleep(0.01)

    @timeit(level=2)
    def too_fine():
        pass

    @timeit("synced", level=1, barrier=True, sync_device=True)           # no process group, no GPU: both are no-ops
    def synced():
        return 5

    plain_work()
    plain_work()
    too_fine()
    assert synced() == 5
    rep = timers.report(reset=False)
    assert set(rep) == {"synced"}                                        # default level 2 is finer than the timers' level 1
    timers2 = init_timers(log_level=2, use_event=False)
    plain_work()
    too_fine()
    rep = timers2.report()
    assert rep["plain_work"] >= 9.0 and "too_fine" in rep
    with pytest.raises(ValueError):
        with timeit():
            pass
    init_timers(0)


def test_dispatcher_names_of_the_reference_are_understood():
    import pytest

    from steptronoss_b200.parallel.ep_dispatcher import AllToAllDispatcher, build_dispatcher

    for name in ("alltoall", "token", "Token"):
        assert isinstance(build_dispatcher(name, "EP", 8), AllToAllDispatcher)
    with pytest.raises(ValueError, match="unknown MoE dispatcher"):
        build_dispatcher("carrier-pigeon", "EP", 8)


def test_retry_on_sync_and_async_with_backoff():
    import asyncio

    import pytest

    from steptronoss_b200.utils.general import retry_on

    seen = []

    @retry_on((ValueError,), retries=3, delay=0.001, on_retry=lambda e, n: seen.append((str(e), n)))
    def flaky(box=[0]):
        box[0] += 1
        if box[0] < 3:
            raise ValueError(f"try {box[0]}")
        return box[0]

    assert flaky() == 3 and seen == [("try 1", 0), ("try 2", 1)]

    @retry_on((ValueError,), retries=1, delay=0.001)
    def hopeless():
        raise ValueError("always")

    with pytest.raises(ValueError, match="always"):
        hopeless()

    @retry_on((ValueError,), retries=2, delay=0.001)
    def other_error():
        raise KeyError("not retried")

    with pytest.raises(KeyError):
        other_error()

    calls = []

    @retry_on((RuntimeError,), retries=2, delay=0.001)
    async def aflaky():
        calls.append(1)
        if len(calls) < 2:
            raise RuntimeError("once")
        return "ok"

    assert asyncio.run(aflaky()) == "ok" and len(calls) == 2


def test_metric_holder_fork_and_disable_and_inverse_reshape_op():
    import torch

    from steptronoss_b200.checkpointing.reshape_ops import ColumnParallel, Inverse
    from steptronoss_b200.utils.metrics import GroupMetric, Metric, MetricHolder

    h = MetricHolder()
    h.loss = Metric().mean("time")
    h.per_layer = GroupMetric().mean("time")
    h.loss.add(1.0)
    h.per_layer.add(2.0, subname="layer0")
    with h.fork():                                               # e.g. an evaluation pass in the middle of an interval
        h.loss.add(100.0)
        assert float(h.loss.reduce()) == 100.0
    with h.disable():
        h.loss.add(1000.0)                                       # dropped
    h.loss.add(3.0)
    out = h.reduce_all()
    assert float(out["loss"]) == 2.0 and float(out["per_layer/layer0"]) == 2.0

    w = torch.arange(12.0).reshape(4, 3)
    merged = Inverse(ColumnParallel()).forward({"w": list(w.chunk(2))})      # the backward of a split is the concatenation
    assert torch.equal(merged["w"], w)
    assert [t.tolist() for t in Inverse(ColumnParallel()).backward({"w": w})["w"]] == [w.tolist()]


def test_seeding_helper_and_rng_tracker_names():
    import random

    import numpy as np

    from steptronoss_b200 import initialize
    from steptronoss_b200.parallel.random import CudaRNGStatesTracker, get_cuda_rng_tracker, get_rng_tracker

    draws = []
    for _ in range(2):
        initialize.set_random_seed(5)
        draws.append((random.random(), float(np.random.rand()), float(torch.rand(1))))
    assert draws[0] == draws[1]
    assert get_cuda_rng_tracker() is get_rng_tracker() and isinstance(get_rng_tracker(), CudaRNGStatesTracker)
    assert callable(initialize.mtp_initialize) and callable(initialize.set_mpu_random_seed)
