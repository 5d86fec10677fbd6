"""Tick-based simulation of rollout flow control, for choosing ``prompt_per_iter``, ``max_untrained_prompts``,
``max_staleness`` and the generation concurrency without real models.

It answers the same question as ``steptronoss/core/generators/flow_controller_simulator.py`` in the reference and
renders comparable timelines.  Model: prompt ``i`` needs ``genables[i]`` ticks of inference, a training step needs
``train_cost`` ticks, inference runs at most ``max_concurrent`` prompts at once (``None`` = unlimited).

* ``on-policy``: batch ``k`` is generated on weights ``k`` -> inference idles during training and vice versa;
* ``one-step-off``: batch ``k`` may be generated on weights ``k-1`` -> the next batch is generated while the
  current one trains;
* ``fully-async``: prompts start whenever a slot is free, fewer than ``max_untrained_prompts`` + 1 are
  outstanding (running or finished but untrained) and the weights are not updated while a running prompt
  would become older than ``max_staleness`` versions; a training step starts as soon as ``prompt_per_iter``
  finished prompts are waiting.

    python -m steptronoss_b200.generators.flow_controller_simulator render --strategy fully-async \\
        --prompt_per_iter 2 --train_cost 3 --genables 1,2,3,4,1,2,3,4 --max_untrained_prompts 8 \\
        --max_staleness 1 --max_concurrent 4

How to read the output
----------------------
``Train:``  blank = idle, ``T`` = training, digit = a *yield*: that many prompts are handed to a step starting at
this tick.  ``Infer:`` blank = idle, digit = prompts running (``+`` for ten or more), ``Y`` = the tick of a yield
while inference is idle.  One ``Yield k`` line per training step lists what was still running at that moment as
``id(done/total)`` (``trunc[...]``: these prompts straddle a weight update) and the prompts handed over
(``yield[...]``, with the weight version each was generated on).  ``Block`` lines (grouped strategies) give, per
group, the version it asked for and when its generation started and ended.

Besides the numbers, the module offers what is needed to check the real controllers against this model:
:class:`SimulatedGenableItem` / :class:`SimulatedFlowDataloader` are prompts whose generation takes their cost in
(scaled) wall-clock ticks, so a :class:`~steptronoss_b200.generators.flow_controller.FlowController` can be driven
with the very cost sequence that was simulated (``tests/test_flow_controller.py``).
"""
from __future__ import annotations

import argparse
import asyncio
from collections.abc import Sequence
from dataclasses import dataclass, field

from ..data.nextable import Nextable
from ..generation.base_generatable import TrainableItem

STRATEGIES = ("on-policy", "one-step-off", "fully-async")


# --------------------------------------------------------------------------------------- simulated workload
class SimulatedGenableItem(TrainableItem):
    """A prompt whose generation costs ``infer_cost`` ticks of ``tick_seconds`` and yields one trajectory."""

    tick_seconds = 0.02

    def __init__(self, infer_cost: int, item_id: int, meta: dict | None = None):
        super().__init__()
        self.infer_cost, self.item_id = int(infer_cost), int(item_id)
        if meta:
            self.meta.update(meta)

    def fingerprint(self) -> str:
        return f"sim-{self.item_id}-{self.infer_cost}"

    async def generate(self):
        await asyncio.sleep(self.infer_cost * self.tick_seconds)
        return self.item_id

    async def generate_for_train(self):
        from ..exp.rl import EnvTrajectory

        await asyncio.sleep(self.infer_cost * self.tick_seconds)
        return [EnvTrajectory(trajectory=[self.item_id], is_gen_mask=[1], raw_reward=0.0,
                              meta={"item_id": self.item_id, "infer_cost": self.infer_cost,
                                    "scheduled_version": self.meta.get("scheduled_version")})]


class SimulatedFlowDataloader(Nextable):
    """Serves one :class:`SimulatedGenableItem` per cost, in order; resumable."""

    def __init__(self, infer_costs: Sequence[int]):
        self.costs = [int(c) for c in infer_costs]
        self.cursor = 0

    def __next__(self) -> SimulatedGenableItem:
        if self.cursor >= len(self.costs):
            raise StopIteration
        item = SimulatedGenableItem(self.costs[self.cursor], self.cursor)
        self.cursor += 1
        return item

    def state_dict(self) -> dict:
        return {"cursor": self.cursor}

    def load_state_dict(self, state_dict: dict) -> None:
        self.cursor = int(state_dict["cursor"])


# --------------------------------------------------------------------------------------- what a run records
@dataclass(frozen=True)
class PromptTrace:
    """Life of one prompt: when it was started, on which weights, when it finished, which step trained on it."""
    prompt: int
    cost: int
    version: int
    start_tick: int
    end_tick: int
    step: int = -1


@dataclass(frozen=True)
class FlowSimulationBlock:
    """One group of the grouped strategies: the prompts of a training step and the weights they asked for."""
    index: int
    prompts: tuple
    required_version: int
    start_tick: int
    end_tick: int

    @property
    def prompt_count(self) -> int:
        return len(self.prompts)


@dataclass(frozen=True)
class YieldSnapshot:
    """The moment a batch is handed to training: what is still running (id, ticks done, ticks total), what goes."""
    step: int
    tick: int
    running: tuple
    yielded: tuple
    versions: tuple


@dataclass
class TrainBatch:
    step: int
    start_tick: int
    prompts: list
    versions: list
    """weight version each prompt of the batch was generated on"""

    @property
    def staleness(self) -> int:
        return max(self.step - v for v in self.versions) if self.versions else 0


# the reference's names for the two records of the fully asynchronous strategy
FullyAsyncPromptTrace = PromptTrace
FullyAsyncTrainBatch = TrainBatch


@dataclass
class FlowSimulationResult:
    strategy: str
    genables: list = field(default_factory=list)
    train_cost: int = 0
    train_line: list = field(default_factory=list)
    infer_line: list = field(default_factory=list)
    batches: list = field(default_factory=list)
    snapshots: list = field(default_factory=list)
    traces: list = field(default_factory=list)
    blocks: list = field(default_factory=list)

    @property
    def ticks(self) -> int:
        return len(self.train_line)

    @property
    def train_idle(self) -> float:
        return sum(1 for c in self.train_line if c == " ") / max(self.ticks, 1)

    @property
    def infer_idle(self) -> float:
        return sum(1 for c in self.infer_line if c in " Y") / max(self.ticks, 1)

    @property
    def max_staleness(self) -> int:
        return max((b.staleness for b in self.batches), default=0)

    @property
    def step_intervals(self) -> list:
        """Ticks between the starts of consecutive training steps (the iteration time seen by the trainer)."""
        starts = [b.start_tick for b in self.batches]
        return [b - a for a, b in zip(starts, starts[1:])]

    def render(self) -> str:
        versions = [b.step for b in self.batches]
        lines = [f"Strategy {self.strategy} | Versions {versions} | ticks {self.ticks} | train idle {self.train_idle:.0%} | "
                 f"infer idle {self.infer_idle:.0%} | max staleness {self.max_staleness}",
                 f"Genables {self.genables} | TrainCost {self.train_cost}",
                 "Train: " + "".join(self.train_line), "Infer: " + "".join(self.infer_line)]
        for blk in self.blocks:
            lines.append(f"Block {blk.index}: prompts {list(blk.prompts)} need version {blk.required_version}, "
                         f"generated t={blk.start_tick}..{blk.end_tick}")
        for snap in self.snapshots:
            trunc = ", ".join(f"{p}({done}/{total})" for p, done, total in snap.running)
            given = ", ".join(f"{p}@v{v}" for p, v in zip(snap.yielded, snap.versions))
            lines.append(f"Yield {snap.step} @t={snap.tick}: trunc[{trunc}] yield[{given}]")
        return "\n".join(lines)

    def __str__(self) -> str:
        return self.render()


# --------------------------------------------------------------------------------------- the simulator
class FlowControllerSimulator:
    """``FlowControllerSimulator(flow_cfg).simulate(costs, train_cost)``; ``flow_cfg`` is the same config object the
    real controllers take (``async_strategy``, ``prompt_per_iter`` and, for fully-async, the two limits)."""

    def __init__(self, flow_cfg):
        self.cfg = flow_cfg
        self.strategy = flow_cfg.async_strategy
        if self.strategy not in STRATEGIES:
            raise ValueError(f"unknown strategy {self.strategy!r}; choose from {STRATEGIES}")
        self.prompt_per_iter = int(flow_cfg.prompt_per_iter)
        self.max_untrained = getattr(flow_cfg, "max_untrained_prompts", None)
        self.max_staleness = getattr(flow_cfg, "max_staleness", None)
        if self.strategy == "fully-async":
            if self.max_untrained is None or self.max_staleness is None:
                raise ValueError("fully-async requires max_untrained_prompts and max_staleness")
            if self.max_untrained + 1 < self.prompt_per_iter:
                raise ValueError("fully-async deadlocks when max_untrained_prompts + 1 < prompt_per_iter")

    @staticmethod
    def build_dataloader(infer_costs: Sequence[int]) -> SimulatedFlowDataloader:
        return SimulatedFlowDataloader(infer_costs)

    def required_version(self, block_index: int) -> int:
        """Weights a group waits for under the grouped strategies."""
        lead = 1 if self.strategy == "one-step-off" else 0
        return max(block_index - lead, 0)

    def simulate(self, infer_costs: Sequence[int], train_cost: int, max_concurrent: int | None = None,
                 max_ticks: int = 1_000_000) -> FlowSimulationResult:
        strategy, ppi = self.strategy, self.prompt_per_iter
        cap = max_concurrent if max_concurrent else 10 ** 9
        costs = [int(c) for c in infer_costs]
        n_steps = len(costs) // ppi
        res = FlowSimulationResult(strategy, genables=list(costs), train_cost=int(train_cost))
        next_prompt = 0                    # next prompt of the source
        running: dict = {}                 # prompt -> [remaining ticks, version it runs on, start tick]
        ready: list = []                   # finished, untrained: (prompt, version)
        finished: dict = {}                # prompt -> (version, start tick, end tick)
        version = 0                        # weights the inference side serves
        train_left, step = 0, 0            # ticks left of the running step; steps started so far
        pending_update = False             # a finished step whose weights wait for stale prompts to drain
        trained_in: dict = {}
        for tick in range(max_ticks):
            if step >= n_steps and train_left == 0 and not pending_update:
                break
            # ---- a training step that just finished publishes its weights
            if pending_update:
                stale = [v for _, v, _ in running.values() if version + 1 - v > (self.max_staleness or 0)]
                if strategy != "fully-async" or not stale:
                    version += 1
                    pending_update = False

            # ---- dispatch prompts to inference
            def may_start(p: int) -> bool:
                block = p // ppi
                if block >= n_steps or len(running) >= cap:
                    return False
                if strategy != "fully-async":
                    return version >= self.required_version(block)
                return len(running) + len(ready) <= self.max_untrained and not pending_update

            while next_prompt < len(costs) and may_start(next_prompt):
                running[next_prompt] = [costs[next_prompt], version, tick]
                next_prompt += 1
            # ---- start a training step
            mark = " "
            if train_left == 0 and not pending_update and step < n_steps:
                if strategy == "fully-async":
                    can = len(ready) >= ppi
                    take = ready[:ppi]
                else:
                    want = set(range(step * ppi, (step + 1) * ppi))
                    take = [r for r in ready if r[0] in want]
                    can = len(take) == ppi and version >= step
                if can:
                    for r in take:
                        ready.remove(r)
                        trained_in[r[0]] = step
                    res.batches.append(TrainBatch(step, tick, [p for p, _ in take], [v for _, v in take]))
                    res.snapshots.append(YieldSnapshot(
                        step, tick, tuple((p, costs[p] - left, costs[p]) for p, (left, _, _) in sorted(running.items())),
                        tuple(p for p, _ in take), tuple(v for _, v in take)))
                    train_left, step = train_cost, step + 1
                    mark = str(len(take)) if len(take) < 10 else "+"
            # ---- one tick of work
            if running:
                res.infer_line.append(str(len(running)) if len(running) < 10 else "+")
            else:
                res.infer_line.append("Y" if mark != " " else " ")
            for p in list(running):
                running[p][0] -= 1
                if running[p][0] <= 0:
                    _, v, t0 = running.pop(p)
                    ready.append((p, v))
                    finished[p] = (v, t0, tick + 1)
            if train_left > 0:
                res.train_line.append(mark if mark != " " else "T")
                train_left -= 1
                if train_left == 0:
                    pending_update = True
            else:
                res.train_line.append(" ")
        res.traces = [PromptTrace(p, costs[p], v, t0, t1, trained_in.get(p, -1)) for p, (v, t0, t1) in sorted(finished.items())]
        if strategy != "fully-async":
            for b in range(n_steps):
                members = [t for t in res.traces if t.prompt // ppi == b]
                if members:
                    res.blocks.append(FlowSimulationBlock(b, tuple(t.prompt for t in members), self.required_version(b),
                                                          min(t.start_tick for t in members),
                                                          max(t.end_tick for t in members)))
        return res


class _Cfg:
    """Plain holder with the attributes of the flow-controller configs."""

    def __init__(self, **kw):
        self.max_untrained_prompts = self.max_staleness = None
        for k, v in kw.items():
            setattr(self, k, v)


def simulate_flow_controller(strategy: str, prompt_per_iter: int, train_cost: int, genables: Sequence[int],
                             max_untrained_prompts: int | None = None, max_staleness: int | None = None,
                             max_concurrent: int | None = None, max_ticks: int = 1_000_000) -> FlowSimulationResult:
    """One call: build the config, simulate, return the result."""
    if strategy not in STRATEGIES:
        raise ValueError(strategy)
    cfg = _Cfg(async_strategy=strategy, prompt_per_iter=prompt_per_iter, max_untrained_prompts=max_untrained_prompts,
               max_staleness=max_staleness)
    return FlowControllerSimulator(cfg).simulate(_normalize_genables(genables), train_cost, max_concurrent, max_ticks)


def _normalize_genables(genables) -> list:
    """``"1,2,3"``, ``[1, 2, 3]`` or a single number (one prompt) -> list of positive ints."""
    if isinstance(genables, (int, float)):
        genables = [genables]
    elif isinstance(genables, str):
        genables = [x for x in genables.replace(" ", "").split(",") if x]
    out = [int(x) for x in genables]
    if any(c <= 0 for c in out):
        raise ValueError("every inference cost must be a positive number of ticks")
    return out


class FlowControllerSimulatorCLI:
    """Command line front: ``render`` prints the timelines, ``compare`` puts the three strategies side by side."""

    @staticmethod
    def render(strategy: str, prompt_per_iter: int, train_cost: int, genables, max_untrained_prompts: int | None = None,
               max_staleness: int | None = None, max_concurrent: int | None = None) -> str:
        return simulate_flow_controller(strategy, prompt_per_iter, train_cost, genables, max_untrained_prompts,
                                        max_staleness, max_concurrent).render()

    @staticmethod
    def compare(prompt_per_iter: int, train_cost: int, genables, max_untrained_prompts: int | None = None,
                max_staleness: int | None = None, max_concurrent: int | None = None) -> str:
        rows = []
        for strategy in STRATEGIES:
            limits = (max_untrained_prompts if max_untrained_prompts is not None else 2 * prompt_per_iter,
                      max_staleness if max_staleness is not None else 1) if strategy == "fully-async" else (None, None)
            r = simulate_flow_controller(strategy, prompt_per_iter, train_cost, genables, limits[0], limits[1],
                                         max_concurrent)
            gaps = r.step_intervals
            rows.append(f"{strategy:13s} ticks {r.ticks:6d} | train idle {r.train_idle:4.0%} | infer idle {r.infer_idle:4.0%} | "
                        f"max staleness {r.max_staleness} | mean step interval "
                        f"{(sum(gaps) / len(gaps)) if gaps else 0:.1f}")
        return "\n".join(rows)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description="Rollout flow-control timelines without real models.")
    sub = ap.add_subparsers(dest="command")
    for name in ("render", "compare"):
        sp = sub.add_parser(name)
        if name == "render":
            sp.add_argument("--strategy", required=True, choices=list(STRATEGIES))
        sp.add_argument("--prompt_per_iter", type=int, required=True)
        sp.add_argument("--train_cost", type=int, required=True)
        sp.add_argument("--genables", required=True, help="comma-separated inference cost of every prompt, in order")
        sp.add_argument("--max_untrained_prompts", type=int)
        sp.add_argument("--max_staleness", type=int)
        sp.add_argument("--max_concurrent", type=int)
    argv = list(argv) if argv is not None else None
    import sys

    raw = sys.argv[1:] if argv is None else argv
    if raw and raw[0] not in ("render", "compare", "-h", "--help"):
        raw = ["render"] + list(raw)           # the command may be left out
    a = ap.parse_args(raw)
    if a.command == "compare":
        print(FlowControllerSimulatorCLI.compare(a.prompt_per_iter, a.train_cost, a.genables, a.max_untrained_prompts,
                                                 a.max_staleness, a.max_concurrent))
    else:
        print(FlowControllerSimulatorCLI.render(a.strategy, a.prompt_per_iter, a.train_cost, a.genables,
                                                a.max_untrained_prompts, a.max_staleness, a.max_concurrent))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
