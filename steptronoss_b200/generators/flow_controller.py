"""Rollout scheduling between the trainer and the inference replicas.

Behaviour follows ``steptronoss/core/generators/flow_controller.py:22-505``.  World rank 0 schedules prompts
through a :class:`~steptronoss_b200.utils.rl_utils.PersistentFlow` with three stages::

    source --> pre_gen --(generation + callbacks)--> pre_train --> trainer

* :class:`SimpleFlowController` (``on-policy`` / ``one-step-off``): ``pre_gen`` holds groups
  ``need_version(v), prompt x prompt_per_iter, train``; a group is held until the replicas serve weight version
  ``v`` and is closed when all its prompts have returned.  ``on-policy`` runs group ``k`` on version ``k``;
  ``one-step-off`` lets group ``k`` run on version ``k-1`` so that generation overlaps the previous training
  step.
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
            for ack_id in self._handed_out:
                self.flow["pre_train"].ack(ack_id)
            self._handed_out.clear()
            cv = getattr(self, "_cv", None)
            if cv is not None:
                with cv:
                    cv.notify_all()


class SimpleFlowController(FlowController):
    """Group-at-a-time scheduling (``on-policy`` and ``one-step-off``).

    A *group* is the ``prompt_per_iter`` prompts of one training iteration.  In the durable ``pre_gen`` stage a
    group is written as ``need_version(v)``, its prompts, ``train``; group ``k`` asks for weight version
    ``max(k - lead, 0)`` and may be written once ``k - lead <= train_weight_version + 1``, where ``lead`` is how
    many groups generation may run ahead of training (0 on-policy, 1 one-step-off).

    One *conductor* thread owns the stage: it writes the groups that have become admissible, holds a group at its
    ``need_version`` marker until the replicas serve that version, submits the prompts, and moves the ``train``
    marker downstream when the last prompt of the group has returned.  Everything waits on one condition
    variable (the flow lock), which weight syncs, finished prompts and acknowledgements notify.
    """

    LEAD = {"on-policy": 0, "one-step-off": 1}

    def __init__(self, flow_cfg, generator=None, deploy_fn=None):
        if flow_cfg.async_strategy not in self.LEAD:
            raise ValueError(f"SimpleFlowController schedules {sorted(self.LEAD)}, not {flow_cfg.async_strategy!r}")
        self.cfg = flow_cfg
        self.lead = self.LEAD[flow_cfg.async_strategy]
        self.generator, self.deploy_fn = generator, deploy_fn
        self.infer_weight_version = self.train_weight_version = -1
        self._handed_out: list = []
        self.source_exhausted = False

    # ------------------------------------------------------------------ life cycle
    def start(self, dataloader, model, state_dict: dict | None = None):
        self.model = model
        if PM.world_rank != 0:
            return
        self.generator = self._build_generator()
        self.flow = PersistentFlow(source=PersistentSource(nextable=dataloader), pre_gen=PersistentQueue(),
                                   pre_train=PersistentQueue())
        self._cv = Condition(self.flow.lock)
        self._load_state_dict(state_dict)
        self.flow.meta.setdefault("groups_planned", 0)
        Thread(target=self._conduct, name="rollout-conductor", daemon=True).start()

    def state_dict(self) -> dict:
        if PM.world_rank != 0:
            return {}
        return {"controller_type": "grouped", "train_weight_version": self.train_weight_version,
                "infer_weight_version": self.infer_weight_version, "flow": self.flow.state_dict()}

    def _load_state_dict(self, state_dict):
        if PM.world_rank != 0 or not state_dict:
            return
        # the replicas of a resumed job serve nothing yet; the trainer's version is whatever was saved
        self.infer_weight_version = -1
        self.train_weight_version = state_dict.get("train_weight_version", -1)
        saved = state_dict.get("flow")
        if saved is not None:
            self.flow.load_state_dict(saved)
            logger.info(f"rollout flow restored: {self.flow}")

    # ------------------------------------------------------------------ conductor (holds the flow lock)
    def _write_admissible_groups(self) -> None:
        pre_gen, source, meta = self.flow["pre_gen"], self.flow["source"], self.flow.meta
        while not self.source_exhausted and meta["groups_planned"] - self.lead <= self.train_weight_version + 1:
            wanted = max(meta["groups_planned"] - self.lead, 0)
            prompts = []
            try:
                for _ in range(self.cfg.prompt_per_iter):
                    prompts.append(source.pop())
            except StopIteration:
                # an incomplete last group is still written, so that a snapshot keeps its prompts; without its
                # closing marker it is never handed to the trainer
                self.source_exhausted = True
            pre_gen.put(PersistentFlow.Signal("need_version", version=wanted), *prompts)
            if not self.source_exhausted:
                pre_gen.put(PersistentFlow.Signal("train"))
                meta["groups_planned"] += 1

    def _conduct(self) -> None:
        cv, pre_gen, pre_train = self._cv, self.flow["pre_gen"], self.flow["pre_train"]
        group = {"outstanding": 0, "version_marker": None}
        held = None                                # an entry taken from pre_gen that cannot be acted on yet

        def prompt_returned(genable, generated):
            try:
                failed = isinstance(generated, Exception)
                if failed and not self.cfg.genable_allow_errors:
                    raise generated
                with cv:
                    pre_train.put([] if failed else generated)
                    pre_gen.ack(genable.meta.pop("pre_gen_id"))
            finally:
                with cv:
                    group["outstanding"] -= 1
                    cv.notify_all()

        with cv:
            while True:
                self._write_admissible_groups()
                if held is None:
                    if len(pre_gen) == 0:
                        cv.wait(timeout=self.poll_s)
                        continue
                    held = pre_gen.get()
                entry_id, entry = held
                if not isinstance(entry, PersistentFlow.Signal):
                    entry.meta["pre_gen_id"] = entry_id
                    group["outstanding"] += 1
                    self.generator.submit_with_callback(entry, for_train=True, callback=prompt_returned)
                elif entry.name == "need_version":
                    if self.infer_weight_version < entry["version"]:
                        cv.wait(timeout=self.poll_s)
                        continue
                    group["version_marker"] = entry_id     # acknowledged together with the group's closing marker
                elif entry.name == "train":
                    if group["outstanding"] > 0:
                        cv.wait(timeout=self.poll_s)
                        continue
                    pre_train.put(entry)
                    if group["version_marker"] is not None:
                        pre_gen.ack(group["version_marker"])
                        group["version_marker"] = None
                    pre_gen.ack(entry_id)
                    cv.notify_all()
                held = None

    # ------------------------------------------------------------------ trainer side
    def get_train_samples(self) -> list:
        """The trajectories of one training iteration.  Asking for them is what announces the next weight version:
        the replicas are brought up to date first, which releases the group that waits for it."""
        self.train_weight_version += 1
        self.sync_weight()
        if PM.world_rank != 0:
            return []
        trajectories: list = []
        pre_train = self.flow["pre_train"]
        with self._cv:
            while True:
                if len(pre_train) == 0:
                    self._cv.wait(timeout=self.poll_s)
                    continue
                taken_id, payload = pre_train.get()
                self._handed_out.append(taken_id)
                if isinstance(payload, PersistentFlow.Signal):
                    if payload.name == "train":
                        return trajectories
                    continue
                prompt_id = uuid4().hex                     # trajectories of one prompt share it (group baselines)
                for traj in payload:
                    traj.prompt_id = prompt_id
                trajectories.extend(payload)


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
        self._handed_out: list = []
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
                    self._handed_out.append(ack_id)
                    prompt_id = str(uuid4())
                    for t in trajs:
                        t.prompt_id = prompt_id
                    trajectories.extend(trajs)
                self._cv.notify_all()
        return trajectories
