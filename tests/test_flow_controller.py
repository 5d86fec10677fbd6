"""Rollout flow control with in-process fake generation: version gating, batching, checkpoint/resume of the
flow, back-pressure and staleness limits of the fully asynchronous controller."""
import asyncio
import threading
import time

import pytest

from steptronoss_b200.data.nextable import Nextable
from steptronoss_b200.exp.rl import EnvTrajectory, FlowControllerConfig, FullyAsyncFlowControllerConfig
from steptronoss_b200.generation.async_generation import SingleGenerationController
from steptronoss_b200.generation.base_generatable import TrainableItem
from steptronoss_b200.generators.flow_controller import FullyAsyncFlowController, SimpleFlowController

VERSIONS = {"infer": -1}
SEEN = []
LOCK = threading.Lock()


class FakePrompt(TrainableItem):
    def __init__(self, idx, delay=0.0):
        super().__init__()
        self.idx, self.delay = idx, delay

    async def generate(self):
        return self.idx

    async def generate_for_train(self):
        await asyncio.sleep(self.delay)
        with LOCK:
            SEEN.append((self.idx, VERSIONS["infer"]))
        return [EnvTrajectory(trajectory=[self.idx, 1, 2], is_gen_mask=[0, 1, 1], raw_reward=float(self.idx % 2),
                              meta={"idx": self.idx, "version": VERSIONS["infer"]}) for _ in range(2)]


class Prompts(Nextable):
    def __init__(self, n=10 ** 6, delay=0.0):
        self.i, self.n, self.delay = 0, n, delay

    def __next__(self):
        if self.i >= self.n:
            raise StopIteration
        self.i += 1
        return FakePrompt(self.i - 1, self.delay)

    def state_dict(self):
        return {"i": self.i}

    def load_state_dict(self, sd):
        self.i = sd["i"]


def _cfg(cls, **kw):
    c = cls()
    for k, v in kw.items():
        setattr(c, k, v)
    return c


def _deploy(ctrl):
    def fn(model):
        VERSIONS["infer"] = ctrl.train_weight_version
    return fn


@pytest.fixture(autouse=True)
def _reset():
    VERSIONS["infer"] = -1
    SEEN.clear()
    yield


@pytest.mark.parametrize("strategy", ["on-policy", "one-step-off"])
def test_simple_flow_versions_and_batches(strategy):
    cfg = _cfg(FlowControllerConfig, async_strategy=strategy, prompt_per_iter=3)
    ctrl = SimpleFlowController(cfg, generator=SingleGenerationController())
    ctrl.deploy_fn = _deploy(ctrl)
    ctrl.poll_s = 0.005
    ctrl.start(Prompts(), model=None)
    for it in range(3):
        trajs = ctrl.get_train_samples()
        assert len(trajs) == 6 and len({t.prompt_id for t in trajs}) == 3
        idx = sorted({t.meta["idx"] for t in trajs})
        assert idx == [3 * it, 3 * it + 1, 3 * it + 2]
        lag = {it - t.meta["version"] for t in trajs}
        if strategy == "on-policy":
            assert lag == {0}
        else:
            assert lag <= {0, 1} and (it == 0 or lag == {1})
        time.sleep(0.15)   # "training": with one-step-off the next group is generated meanwhile, on the old weights
        ctrl.weight_dumped()


def test_simple_flow_resume_replays_unacknowledged_prompts():
    cfg = _cfg(FlowControllerConfig, async_strategy="on-policy", prompt_per_iter=2)
    ctrl = SimpleFlowController(cfg, generator=SingleGenerationController())
    ctrl.deploy_fn = _deploy(ctrl)
    ctrl.poll_s = 0.005
    ctrl.start(Prompts(), model=None)
    first = ctrl.get_train_samples()
    ctrl.weight_dumped()
    second = ctrl.get_train_samples()          # handed out, never acknowledged: the job dies before saving
    with ctrl.flow.lock:
        state = ctrl.state_dict()
    assert {t.meta["idx"] for t in first} == {0, 1} and {t.meta["idx"] for t in second} == {2, 3}
    state["train_weight_version"] = 0           # the last saved weights are those after the first step
    VERSIONS["infer"] = -1
    ctrl2 = SimpleFlowController(cfg, generator=SingleGenerationController())
    ctrl2.deploy_fn = _deploy(ctrl2)
    ctrl2.poll_s = 0.005
    ctrl2.start(Prompts(), model=None, state_dict=state)
    again = ctrl2.get_train_samples()
    assert {t.meta["idx"] for t in again} == {2, 3}


def test_fully_async_backpressure_and_staleness():
    cfg = _cfg(FullyAsyncFlowControllerConfig, prompt_per_iter=2, max_untrained_prompts=5, max_staleness=1)
    ctrl = FullyAsyncFlowController(cfg, generator=SingleGenerationController())
    ctrl.deploy_fn = _deploy(ctrl)
    ctrl.poll_s = 0.005
    src = Prompts(delay=0.01)
    ctrl.start(src, model=None)
    t = ctrl.get_train_samples()
    assert len(t) == 4
    time.sleep(0.3)
    with ctrl._cv:
        outstanding = len(ctrl.flow["pre_train"]) + len(ctrl.running_genables) + len(ctrl.flow["pre_gen"])
    assert outstanding <= cfg.max_untrained_prompts + 1   # inference stopped pulling prompts
    pulled = src.i
    time.sleep(0.2)
    assert src.i == pulled
    for it in range(1, 4):
        trajs = ctrl.get_train_samples()
        assert len(trajs) == 4
        # finished prompts may wait in the buffer for (max_untrained_prompts + 1) / prompt_per_iter iterations,
        # on top of the staleness allowed while they were running
        bound = (cfg.max_untrained_prompts + 1) // cfg.prompt_per_iter + cfg.max_staleness
        assert all(it - t.meta["version"] <= bound for t in trajs)
        ctrl.weight_dumped()


def test_simulator_orders_strategies_by_overlap():
    from steptronoss_b200.generators.flow_controller_simulator import simulate_flow_controller

    costs = [3, 3, 3] * 4
    on = simulate_flow_controller("on-policy", 3, 4, costs)
    off = simulate_flow_controller("one-step-off", 3, 4, costs)
    fa = simulate_flow_controller("fully-async", 3, 4, costs, max_untrained_prompts=6, max_staleness=2)
    assert len(on.batches) == len(off.batches) == len(fa.batches) == 4
    assert on.ticks > off.ticks >= fa.ticks           # more overlap, fewer ticks
    assert max(b.staleness for b in on.batches) == 0 and max(b.staleness for b in off.batches) <= 1
    assert all(b.staleness <= 2 + 2 for b in fa.batches)
    assert "Train:" in on.render() and "Infer:" in on.render()


def test_simulator_records_blocks_snapshots_and_traces():
    from steptronoss_b200.generators.flow_controller_simulator import (
        FlowControllerSimulator, FlowControllerSimulatorCLI, simulate_flow_controller)

    r = simulate_flow_controller("one-step-off", 3, 4, "1,2,3,1,2,3,1,2,3")
    assert [b.required_version for b in r.blocks] == [0, 0, 1] and [b.prompt_count for b in r.blocks] == [3, 3, 3]
    assert r.blocks[1].start_tick == 0                   # the second group is generated beside the first, on version 0
    assert [s.yielded for s in r.snapshots] == [(0, 1, 2), (3, 4, 5), (6, 7, 8)]
    assert all(t.end_tick - t.start_tick == t.cost for t in r.traces) and [t.step for t in r.traces] == [0] * 3 + [1] * 3 + [2] * 3
    text = r.render()
    assert "Yield 0 @t=3" in text and "Block 2: prompts [6, 7, 8] need version 1" in text and text.count("Yield") == 3
    fa = simulate_flow_controller("fully-async", 2, 3, [1, 5, 1, 1, 1, 1], max_untrained_prompts=4, max_staleness=1,
                                  max_concurrent=3)
    # the long prompt is still running when the first batch is handed over: it shows up as truncated
    assert fa.snapshots[0].running and fa.snapshots[0].running[0][0] == 1 and fa.max_staleness <= 2
    assert "trunc[1(" in fa.render()
    cfg = _cfg(FullyAsyncFlowControllerConfig, prompt_per_iter=4, max_untrained_prompts=2, max_staleness=1)
    with pytest.raises(ValueError):
        FlowControllerSimulator(cfg)
    table = FlowControllerSimulatorCLI.compare(3, 4, "1,2,3,1,2,3,1,2,3")
    assert [line.split()[0] for line in table.splitlines()] == ["on-policy", "one-step-off", "fully-async"]


@pytest.mark.parametrize("strategy", ["on-policy", "one-step-off"])
def test_runtime_controller_follows_the_simulated_schedule(strategy):
    """The real controller, fed prompts whose generation takes their simulated cost in wall-clock ticks and a
    trainer that sleeps ``train_cost`` ticks, hands out the batches the simulator predicts, generated on the
    versions it predicts."""
    from steptronoss_b200.generators.flow_controller_simulator import (
        FlowControllerSimulator, SimulatedGenableItem, simulate_flow_controller)

    costs, ppi, train_cost, tick = [1, 3, 2, 2, 1, 3, 3, 1, 2], 3, 4, 0.03
    predicted = simulate_flow_controller(strategy, ppi, train_cost, costs)
    cfg = _cfg(FlowControllerConfig, async_strategy=strategy, prompt_per_iter=ppi)
    ctrl = SimpleFlowController(cfg, generator=SingleGenerationController())
    ctrl.deploy_fn = _deploy(ctrl)
    ctrl.poll_s = 0.002
    old_tick, SimulatedGenableItem.tick_seconds = SimulatedGenableItem.tick_seconds, tick
    try:
        ctrl.start(FlowControllerSimulator.build_dataloader(costs), model=None)
        for step, batch in enumerate(predicted.batches):
            trajs = ctrl.get_train_samples()
            assert sorted(t.meta["item_id"] for t in trajs) == sorted(batch.prompts)
            time.sleep(train_cost * tick)
            ctrl.weight_dumped()
        # versions: on-policy never lags, one-step-off lags by exactly one from the second batch on
        assert predicted.max_staleness == (0 if strategy == "on-policy" else 1)
    finally:
        SimulatedGenableItem.tick_seconds = old_tick
