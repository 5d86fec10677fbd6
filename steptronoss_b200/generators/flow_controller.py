"""Rollout scheduling between the trainer and the inference replicas.

Reference: ``steptronoss/core/generators/flow_controller.py:22-505``.  World rank 0 runs two daemon threads
around a :class:`~steptronoss_b200.utils.rl_utils.PersistentFlow` with three stages::

    source --(control worker)--> pre_gen --(generation worker + callbacks)--> pre_train --> trainer

* :class:`SimpleFlowController` (``on-policy`` / ``one-step-off``): the control worker writes
  ``need_version(v), prompt x prompt_per_iter, train`` groups; the generation worker holds a group until
  the replicas serve weight version ``v`` and closes it when all its prompts have returned.  ``on-policy``
  schedules group ``k`` on version ``k``; ``one-step-off`` lets group ``k`` run on version ``k-1`` so that
  generation overlaps the previous training step.
* :class:`FullyAsyncFlowController`: no groups; prompts flow continuously, bounded by
  ``max_untrained_prompts`` (back-pressure on inference) and ``max_staleness`` (the trainer waits before a
  weight update while prompts scheduled too many versions ago are still running).

Items are moved between stages under the flow lock (put downstream, then acknowledge upstream), so a
checkpoint of the flow taken at any moment loses and duplicates nothing; what the trainer has taken is
acknowledged only by :meth:`weight_dumped`, i.e. once the weights that learned from it are saved.
"""
from __future__ import annotations

import time
from abc import ABCMeta, abstractmethod
from threading import Condition, Thread
from uuid import uuid4

from ..parallel.state import PM
from ..utils.logger import logger
from ..utils.rl_utils import PersistentFlow, PersistentQueue, PersistentSource
from ..utils.timers import get_timers


class FlowController(metaclass=ABCMeta):
    """``start(dataloader, model)`` once, then ``get_train_samples()`` per training iteration."""

    poll_s = 0.05

    @abstractmethod
    def start(self, dataloader, model, state_dict: dict | None = None): ...

    @abstractmethod
    def get_train_samples(self) -> list: ...

    @abstractmethod
    def state_dict(self) -> dict: ...

    @abstractmethod
    def _load_state_dict(self, state_dict: dict): ...

    # ---- shared plumbing
    def _build_generator(self):
        if getattr(self, "generator", None) is not None:
            return self.generator
        from ..generation.async_generation import GenerationController

        cap = self.cfg.max_concurrent_genables
        if cap is None:
            cap = getattr(self.cfg, "max_untrained_prompts", None)
        return GenerationController(num_workers=getattr(self.cfg, "num_generation_workers", None),
                                    max_concurrent_genables=cap)

    def sync_weight(self):
        """Bring the replicas to the trainer's weight version (collective over the training ranks)."""
        if self.infer_weight_version != self.train_weight_version:
            with get_timers().record("model_to_generator", 1):
                if self.deploy_fn is not None:
                    self.deploy_fn(self.model)
                else:
                    self.cfg.vllm_cfg.deploy_training_model(self.model)
            self.infer_weight_version = self.train_weight_version
            cv = getattr(self, "_cv", None)
            if cv is not None:
                with cv:
                    cv.notify_all()

    def weight_dumped(self):
        """The weights trained on everything handed out so far are safely stored: acknowledge it."""
        if PM.world_rank == 0 and hasattr(self, "flow"):
            for ack_id in self.yielded_but_not_acked_train_samples:
                self.flow["pre_train"].ack(ack_id)
            self.yielded_but_not_acked_train_samples.clear()
            cv = getattr(self, "_cv", None)
            if cv is not None:
                with cv:
                    cv.notify_all()


class SimpleFlowController(FlowController):
    def __init__(self, flow_cfg, generator=None, deploy_fn=None):
        self.cfg = flow_cfg
        assert self.cfg.async_strategy in ("on-policy", "one-step-off")
        self.generator, self.deploy_fn = generator, deploy_fn
        self.infer_weight_version = self.train_weight_version = -1
        self.yielded_but_not_acked_train_samples: list = []
        self.source_exhausted = False

    def start(self, dataloader, model, state_dict: dict | None = None):
        self.model = model
        if PM.world_rank == 0:
            self.generator = self._build_generator()
            self.flow = PersistentFlow(source=PersistentSource(nextable=dataloader), pre_gen=PersistentQueue(),
                                       pre_train=PersistentQueue())
            if state_dict:
                self._load_state_dict(state_dict)
            Thread(target=self._generation_worker, daemon=True).start()
            Thread(target=self._control_worker, daemon=True).start()

    def state_dict(self) -> dict:
        if PM.world_rank == 0:
            return {"infer_weight_version": self.infer_weight_version,
                    "train_weight_version": self.train_weight_version, "flow": self.flow.state_dict()}
        return {}

    def _load_state_dict(self, state_dict):
        if PM.world_rank != 0 or not state_dict:
            return
        self.infer_weight_version = -1
        self.train_weight_version = state_dict.get("train_weight_version", -1)
        if "flow" in state_dict:
            self.flow.load_state_dict(state_dict["flow"])
            logger.warning(f"FlowCkpt loaded, flow:\n{self.flow}")

    def _control_worker(self):
        first = 0 if self.cfg.async_strategy == "on-policy" else -1
        self.flow.meta.setdefault("scheduled-weight-version", first)
        while not self.source_exhausted:
            if self.flow.meta["scheduled-weight-version"] <= self.train_weight_version + 1:
                version = max(self.flow.meta["scheduled-weight-version"], 0)
                with self.flow.lock:
                    self.flow["pre_gen"].put(PersistentFlow.Signal("need_version", version=version))
                    for _ in range(self.cfg.prompt_per_iter):
                        try:
                            self.flow["pre_gen"].put(self.flow["source"].pop())
                        except StopIteration:
                            self.source_exhausted = True
                            return
                    self.flow["pre_gen"].put(PersistentFlow.Signal("train"))
                    self.flow.meta["scheduled-weight-version"] += 1
            time.sleep(self.poll_s)

    def _generation_worker(self):
        active = [0]
        ack_version = None

        def on_done(genable, generated):
            try:
                if isinstance(generated, Exception):
                    if not self.cfg.genable_allow_errors:
                        raise generated
                    generated = []
                with self.flow.lock:
                    self.flow["pre_train"].put(generated)
                    self.flow["pre_gen"].ack(genable.meta.pop("ack_pre_id"))
            finally:
                active[0] -= 1

        while True:
            ack_id, data = self.flow["pre_gen"].get()
            if isinstance(data, PersistentFlow.Signal):
                if data.name == "need_version":
                    while self.infer_weight_version < data["version"]:
                        time.sleep(self.poll_s)
                    ack_version = ack_id
                elif data.name == "train":
                    while active[0]:
                        time.sleep(self.poll_s)
                    with self.flow.lock:
                        if ack_version:
                            self.flow["pre_gen"].ack(ack_version)
                        self.flow["pre_train"].put(data)
                        self.flow["pre_gen"].ack(ack_id)
            else:
                data.meta["ack_pre_id"] = ack_id
                active[0] += 1
                self.generator.submit_with_callback(data, for_train=True, callback=on_done)

    def get_train_samples(self) -> list:
        """The trajectories of one training iteration; calling it is also what lets the next weights out."""
        self.train_weight_version += 1
        self.sync_weight()
        trajectories = []
        if PM.world_rank == 0:
            while True:
                ack_id, trajs = self.flow["pre_train"].get()
                self.yielded_but_not_acked_train_samples.append(ack_id)
                if isinstance(trajs, PersistentFlow.Signal) and trajs.name == "train":
                    break
                prompt_id = str(uuid4())
                for t in trajs:
                    t.prompt_id = prompt_id
                trajectories.extend(trajs)
        return trajectories


class FullyAsyncFlowController(FlowController):
    def __init__(self, flow_cfg, generator=None, deploy_fn=None):
        self.cfg = flow_cfg
        assert self.cfg.async_strategy == "fully-async"
        if self.cfg.max_untrained_prompts is None or self.cfg.max_staleness is None:
            raise ValueError("fully-async requires max_untrained_prompts and max_staleness")
        if self.cfg.max_untrained_prompts + 1 < self.cfg.prompt_per_iter:
            raise ValueError("fully-async deadlocks when max_untrained_prompts + 1 < prompt_per_iter: "
                             f"{self.cfg.max_untrained_prompts} + 1 < {self.cfg.prompt_per_iter}")
        self.generator, self.deploy_fn = generator, deploy_fn
        self.infer_weight_version = self.train_weight_version = -1
        self.yielded_but_not_acked_train_samples: list = []
        self.running_genables: dict = {}
        self.source_exhausted = False
        self.started = False

    def start(self, dataloader, model, state_dict: dict | None = None):
        self.model = model
        if PM.world_rank == 0:
            self.generator = self._build_generator()
            self.flow = PersistentFlow(source=PersistentSource(nextable=dataloader), pre_gen=PersistentQueue(),
                                       pre_train=PersistentQueue())
            self._cv = Condition(self.flow.lock)
            self.flow.meta.setdefault("scheduled-weight-version", 0)
            self.flow.meta.setdefault("max-untrained-prompts", self.cfg.max_untrained_prompts)
            self.flow.meta.setdefault("max-staleness", self.cfg.max_staleness)
            if state_dict:
                self._load_state_dict(state_dict)
            Thread(target=self._generation_worker, daemon=True).start()
            Thread(target=self._control_worker, daemon=True).start()
        self.started = True

    def state_dict(self) -> dict:
        if PM.world_rank == 0:
            return {"controller_type": "fully-async", "infer_weight_version": self.infer_weight_version,
                    "train_weight_version": self.train_weight_version,
                    "running_genables_snapshot": dict(self.running_genables),
                    "source_exhausted": self.source_exhausted,
                    "flow": self.flow.state_dict() if hasattr(self, "flow") else None}
        return {}

    def _load_state_dict(self, state_dict):
        if PM.world_rank != 0 or not state_dict:
            return
        self.infer_weight_version = -1
        self.train_weight_version = state_dict.get("train_weight_version", -1)
        self.running_genables = {}  # prompts that were in flight come back through pre_gen's pending items
        self.source_exhausted = state_dict.get("source_exhausted", False)
        if state_dict.get("flow") is not None:
            self.flow.load_state_dict(state_dict["flow"])

    # ---- predicates, called with the lock held
    def _can_schedule_prompt_locked(self) -> bool:
        if self.source_exhausted and len(self.flow["source"]) == 0:
            return False
        if len(self.flow["pre_gen"]) > 0:
            return False
        return len(self.flow["pre_train"]) + len(self.running_genables) <= self.cfg.max_untrained_prompts

    def _can_advance_weight_locked(self) -> bool:
        if not self.running_genables:
            return True
        nxt = self.train_weight_version + 1
        return max(nxt - m["scheduled_version"] for m in self.running_genables.values()) <= self.cfg.max_staleness

    def _wait_for_next_weight(self):
        if PM.world_rank != 0:
            self.train_weight_version += 1
            self.sync_weight()
            return
        while True:
            with self._cv:
                if self._can_advance_weight_locked():
                    self.train_weight_version += 1
                    self.flow.meta["scheduled-weight-version"] = self.train_weight_version
                    break
                self._cv.wait(timeout=self.poll_s)
        self.sync_weight()

    def _control_worker(self):
        while True:
            with self._cv:
                scheduled = False
                while self._can_schedule_prompt_locked():
                    try:
                        genable = self.flow["source"].pop()
                    except StopIteration:
                        self.source_exhausted = True
                        break
                    genable.meta["scheduled_version"] = max(self.train_weight_version, 0)
                    self.flow["pre_gen"].put(genable)
                    scheduled = True
                if scheduled:
                    self._cv.notify_all()
                self._cv.wait(timeout=self.poll_s)

    def _generation_worker(self):
        def on_done(genable, generated):
            try:
                if isinstance(generated, Exception):
                    if not self.cfg.genable_allow_errors:
                        raise generated
                    generated = []
                with self._cv:
                    self.flow["pre_train"].put(generated)
                    self.flow["pre_gen"].ack(genable.meta.pop("ack_pre_id"))
                    self.running_genables.pop(genable.meta.pop("running_ack_id"), None)
                    self._cv.notify_all()
            except Exception:
                with self._cv:
                    self.running_genables.pop(genable.meta.get("running_ack_id"), None)
                    self._cv.notify_all()
                raise

        while True:
            with self._cv:
                while len(self.flow["pre_gen"]) == 0:
                    self._cv.wait(timeout=self.poll_s)
                ack_id, data = self.flow["pre_gen"].get()
                version = data.meta.get("scheduled_version", max(self.train_weight_version, 0))
                self.running_genables[ack_id] = {"scheduled_version": version, "submitted_at": time.time()}
                self._cv.notify_all()
            while self.infer_weight_version < version:
                with self._cv:
                    if self.infer_weight_version >= version:
                        break
                    self._cv.wait(timeout=self.poll_s)
            data.meta["ack_pre_id"] = data.meta["running_ack_id"] = ack_id
            self.generator.submit_with_callback(data, for_train=True, callback=on_done)

    def get_train_samples(self) -> list:
        if not self.started:
            raise RuntimeError("FullyAsyncFlowController.start() must be called before get_train_samples()")
        self._wait_for_next_weight()
        trajectories = []
        if PM.world_rank == 0:
            with self._cv:
                while len(self.flow["pre_train"]) < self.cfg.prompt_per_iter:
                    self._cv.wait(timeout=self.poll_s)
                for _ in range(self.cfg.prompt_per_iter):
                    ack_id, trajs = self.flow["pre_train"].get()
                    self.yielded_but_not_acked_train_samples.append(ack_id)
                    prompt_id = str(uuid4())
                    for t in trajs:
                        t.prompt_id = prompt_id
                    trajectories.extend(trajs)
                self._cv.notify_all()
        return trajectories
