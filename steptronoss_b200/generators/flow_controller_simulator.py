"""Tick-based simulation of rollout flow control, for choosing ``prompt_per_iter``, ``max_untrained_prompts``,
``max_staleness`` and the generation concurrency without real models.

Reference: ``steptronoss/core/generators/flow_controller_simulator.py`` (same question, same timeline
rendering idea).  Model: prompt ``i`` needs ``genables[i]`` ticks of inference, a training step needs
``train_cost`` ticks, inference runs at most ``max_concurrent`` prompts at once (``None`` = unlimited).

* ``on-policy``: batch ``k`` is generated on weights ``k`` -> inference idles during training and vice versa;
* ``one-step-off``: batch ``k`` may be generated on weights ``k-1`` -> the next batch is generated while the
  current one trains;
* ``fully-async``: prompts start whenever a slot is free, fewer than ``max_untrained_prompts`` + 1 are
  outstanding (running or finished but untrained) and the weights are not updated while a running prompt
  would become older than ``max_staleness`` versions; a training step starts as soon as ``prompt_per_iter``
  finished prompts are waiting.

    python -m steptronoss_b200.generators.flow_controller_simulator --strategy fully-async \\
        --prompt_per_iter 2 --train_cost 3 --genables 1,2,3,4,1,2,3,4 --max_untrained_prompts 8 \\
        --max_staleness 1 --max_concurrent 4

Timelines: ``Train:`` blank = idle, ``T`` = training, digit = prompts handed to a step that starts at this
tick; ``Infer:`` blank = idle, digit = prompts running (``+`` for ten or more).
"""
from __future__ import annotations

import argparse
from dataclasses import dataclass, field


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


@dataclass
class FlowSimulationResult:
    strategy: str
    train_line: list = field(default_factory=list)
    infer_line: list = field(default_factory=list)
    batches: list = field(default_factory=list)

    @property
    def ticks(self) -> int:
        return len(self.train_line)

    @property
    def train_idle(self) -> float:
        return sum(1 for c in self.train_line if c == " ") / max(self.ticks, 1)

    @property
    def infer_idle(self) -> float:
        return sum(1 for c in self.infer_line if c == " ") / max(self.ticks, 1)

    def render(self) -> str:
        head = (f"Strategy {self.strategy} | ticks {self.ticks} | train idle {self.train_idle:.0%} | "
                f"infer idle {self.infer_idle:.0%} | max staleness {max((b.staleness for b in self.batches), default=0)}")
        lines = [head, "Train: " + "".join(self.train_line), "Infer: " + "".join(self.infer_line)]
        for b in self.batches:
            lines.append(f"Step {b.step} @t={b.start_tick}: prompts {b.prompts} generated on versions {b.versions}")
        return "\n".join(lines)

    def __str__(self) -> str:
        return self.render()


def simulate_flow_controller(strategy: str, prompt_per_iter: int, train_cost: int, genables: list,
                             max_untrained_prompts: int | None = None, max_staleness: int | None = None,
                             max_concurrent: int | None = None, max_ticks: int = 100000) -> FlowSimulationResult:
    if strategy not in ("on-policy", "one-step-off", "fully-async"):
        raise ValueError(strategy)
    if strategy == "fully-async":
        if max_untrained_prompts is None or max_staleness is None:
            raise ValueError("fully-async requires max_untrained_prompts and max_staleness")
        if max_untrained_prompts + 1 < prompt_per_iter:
            raise ValueError("fully-async deadlocks when max_untrained_prompts + 1 < prompt_per_iter")
    cap = max_concurrent if max_concurrent else 10 ** 9
    costs = list(genables)
    n_steps = len(costs) // prompt_per_iter
    res = FlowSimulationResult(strategy)
    next_prompt = 0                    # next prompt of the source
    running: dict = {}                 # prompt -> [remaining ticks, version it runs on]
    ready: list = []                   # finished, untrained: (prompt, version)
    version = 0                        # weights the inference side serves
    train_left, step = 0, 0            # ticks left of the running step; steps started so far
    pending_update = False             # a finished step whose weights wait for stale prompts to drain
    for tick in range(max_ticks):
        if step >= n_steps and train_left == 0 and not pending_update:
            break
        # ---- a training step that just finished publishes its weights
        if pending_update:
            stale = [v for _, v in running.values() if version + 1 - v > (max_staleness or 0)]
            if strategy != "fully-async" or not stale:
                version += 1
                pending_update = False
        # ---- dispatch prompts to inference
        def may_start(p: int) -> bool:
            batch = p // prompt_per_iter
            if batch >= n_steps or len(running) >= cap:
                return False
            if strategy == "on-policy":
                return version >= batch
            if strategy == "one-step-off":
                return version >= batch - 1
            return len(running) + len(ready) <= max_untrained_prompts and not pending_update

        while next_prompt < len(costs) and may_start(next_prompt):
            running[next_prompt] = [costs[next_prompt], version]
            next_prompt += 1
        # ---- start a training step
        mark = " "
        if train_left == 0 and not pending_update and step < n_steps:
            if strategy == "fully-async":
                can = len(ready) >= prompt_per_iter
                take = ready[:prompt_per_iter]
            else:
                want = set(range(step * prompt_per_iter, (step + 1) * prompt_per_iter))
                take = [r for r in ready if r[0] in want]
                can = len(take) == prompt_per_iter and version >= step
            if can:
                for r in take:
                    ready.remove(r)
                res.batches.append(TrainBatch(step, tick, [p for p, _ in take], [v for _, v in take]))
                train_left, step = train_cost, step + 1
                mark = str(len(take)) if len(take) < 10 else "+"
        # ---- one tick of work
        res.infer_line.append(" " if not running else (str(len(running)) if len(running) < 10 else "+"))
        for p in list(running):
            running[p][0] -= 1
            if running[p][0] <= 0:
                ready.append((p, running.pop(p)[1]))
        if train_left > 0:
            res.train_line.append(mark if mark != " " else "T")
            train_left -= 1
            if train_left == 0:
                pending_update = True
        else:
            res.train_line.append(" ")
    return res


def _parse_genables(text) -> list:
    if isinstance(text, (list, tuple)):
        return [int(x) for x in text]
    return [int(x) for x in str(text).replace(" ", "").split(",") if x]


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description="Render rollout flow-control timelines.")
    ap.add_argument("--strategy", required=True, choices=["on-policy", "one-step-off", "fully-async"])
    ap.add_argument("--prompt_per_iter", type=int, required=True)
    ap.add_argument("--train_cost", type=int, required=True)
    ap.add_argument("--genables", required=True, help="comma-separated inference cost of every prompt, in order")
    ap.add_argument("--max_untrained_prompts", type=int)
    ap.add_argument("--max_staleness", type=int)
    ap.add_argument("--max_concurrent", type=int)
    a = ap.parse_args(argv)
    print(simulate_flow_controller(a.strategy, a.prompt_per_iter, a.train_cost, _parse_genables(a.genables),
                                   a.max_untrained_prompts, a.max_staleness, a.max_concurrent).render())
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
