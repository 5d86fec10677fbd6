"""Native checkpoint layout and resume protocol.

On-disk layout of the reference (``steptronoss/checkpointing/local_checkpoint.py:59-510``,
``checkpointing/utils.py:16-184``), kept unchanged so existing tooling can read it::

    <save_path>/latest_ckpt                       text file: directory of the last COMPLETE checkpoint
    <save_path>/it<N>/TPxx_PPxxx_DPxxx.pt          {"model" | "model0..k", "extra", "rng_state", "scheduler"}
    <save_path>/it<N>/TPxx_PPxxx_DPxxx_OPT.pt      {"optimizer": ...}   (every rank under ZeRO-1)
    <save_path>/it<N>/data.pkl                     dataloader state (rank 0)
    <save_path>/it<N>/<rank>.success               one marker per rank

Model weights are written only by the first data-parallel replica (DP rank 0, or EDP rank 0 for
expert parameters); ``latest_ckpt`` is replaced atomically by whichever rank finishes last, once all
``<rank>.success`` markers exist, so an interrupted save can never be resumed from.  Saving can run
on a background thread (state is first copied to host memory).
"""
from __future__ import annotations

import os
import pickle
import re
import threading

from typing import TypedDict

import torch

from ..config import recur_to_allowed_types
from ..models.module import unwrap_model
from ..parallel.state import PM
from ..utils.dist_utils import broadcast_tensors
from ..utils.logger import logger

_NAME = re.compile(r"TP(\d+)_PP(\d+)_DP(\d+)(_OPT)?\.pt$")


def rank_file_name(opt: bool = False) -> str:
    return f"TP{PM.rank_in('TP'):02d}_PP{PM.rank_in('PP'):03d}_DP{PM.rank_in('DP'):03d}{'_OPT' if opt else ''}.pt"


def analyze_dir(path: str) -> dict:
    """Parallel layout a checkpoint directory was written with (from its file names)."""
    tp = pp = dp = 0
    n = 0
    for f in os.listdir(path):
        m = _NAME.search(f)
        if m and not m.group(4):
            tp, pp, dp = max(tp, int(m.group(1)) + 1), max(pp, int(m.group(2)) + 1), max(dp, int(m.group(3)) + 1)
            n += 1
    return {"tp": tp, "pp": pp, "dp": dp, "files": n}


def optimizer_dp_size(path: str) -> int:
    """Number of data-parallel ranks that wrote optimizer files into ``path`` (0: none did)."""
    dp = 0
    for f in os.listdir(path):
        m = _NAME.search(f)
        if m and m.group(4):
            dp = max(dp, int(m.group(3)) + 1)
    return dp


def _to_cpu(obj):
    if torch.is_tensor(obj):
        return obj.detach().to("cpu", copy=True)
    if isinstance(obj, dict):
        return {k: _to_cpu(v) for k, v in obj.items()}
    if isinstance(obj, (list, tuple)):
        return type(obj)(_to_cpu(v) for v in obj)
    return obj


class CheckpointDict(TypedDict, total=False):
    """What ``load_ckpt`` hands back beside what it loaded in place."""

    iteration: int
    model: list
    optimizer: dict
    scheduler: dict
    data: dict
    extra_info: dict


class Checkpointer:
    def __init__(self, cfg):
        self.cfg = cfg
        self._thread: threading.Thread | None = None
        self._error: BaseException | None = None

    # ------------------------------------------------------------------ paths
    @property
    def save_path(self) -> str:
        return self.cfg.save_path

    def iteration_dir(self, iteration: int, sub_name: str | None = None) -> str:
        d = os.path.join(self.save_path, f"it{iteration}")
        return os.path.join(d, sub_name) if sub_name else d

    def latest(self) -> str | None:
        """Directory named by ``latest_ckpt`` if it exists and is complete."""
        marker = os.path.join(self.save_path, "latest_ckpt")
        if not os.path.exists(marker):
            return None
        path = open(marker).read().strip()
        if not os.path.isabs(path):
            path = os.path.join(self.save_path, path)
        return path if os.path.isdir(path) and self.is_complete(path) else None

    @staticmethod
    def is_complete(path: str, world: int | None = None) -> bool:
        marks = [f for f in os.listdir(path) if f.endswith(".success")]
        if world is None:
            info_file = os.path.join(path, "world_size")
            world = int(open(info_file).read()) if os.path.exists(info_file) else PM.world_size
        return len(marks) >= world

    # ------------------------------------------------------------------ save
    def make_ckpt(self, models, grad_manager, scheduler, dataloader, extra: dict) -> dict:
        files: dict = {}
        keep = getattr(self.cfg, "save_option", None)
        want = (lambda part: True) if keep is None else (lambda part: bool(getattr(keep, part, True)))
        main: dict = {"extra": recur_to_allowed_types(extra)}
        if want("rng_state"):
            main["rng_state"] = PM.get_all_rng()
        first_replica = PM.rank_in("DP") == 0
        edp_first = (PM.rank_in("EDP") == 0) if PM.has("EDP") else first_replica
        if want("model") and (first_replica or edp_first):
            for i, m in enumerate(models):
                sd = unwrap_model(m).state_dict()
                if not first_replica:
                    sd = {k: v for k, v in sd.items() if ".experts." in k}
                elif not edp_first:
                    sd = {k: v for k, v in sd.items() if ".experts." not in k}
                main["model" if len(models) == 1 else f"model{i}"] = _to_cpu(sd)
        if scheduler is not None and want("scheduler"):
            main["scheduler"] = scheduler.state_dict()
        files[rank_file_name()] = main
        if want("optimizer") and grad_manager is not None and hasattr(grad_manager, "state_dict"):
            sharded = getattr(grad_manager, "shard_optimizer", False)
            if sharded or first_replica:
                files[rank_file_name(opt=True)] = _to_cpu(grad_manager.state_dict())
        if PM.world_rank == 0:
            if want("data") and dataloader is not None and hasattr(dataloader, "state_dict"):
                files["data.pkl"] = dataloader.state_dict()
            files["world_size"] = str(PM.world_size)
        return files

    def _write(self, files: dict, path: str, mark_latest: bool = True) -> None:
        for name, obj in files.items():
            dst = os.path.join(path, name)
            tmp = dst + ".tmp"
            if name.endswith(".pt"):
                torch.save(obj, tmp)
            elif name.endswith(".pkl"):
                with open(tmp, "wb") as f:
                    pickle.dump(obj, f)
            else:
                with open(tmp, "w") as f:
                    f.write(str(obj))
            os.replace(tmp, dst)
        open(os.path.join(path, f"{PM.world_rank}.success"), "w").close()
        if mark_latest and self.is_complete(path, PM.world_size):
            marker = os.path.join(self.save_path, "latest_ckpt")
            tmp = marker + f".tmp{PM.world_rank}"
            with open(tmp, "w") as f:
                f.write(path)
            os.replace(tmp, marker)  # atomic: readers see the old or the new pointer, never a partial one
            self._prune()

    def _prune(self) -> None:
        keep = getattr(self.cfg, "keep_last", None)
        if not keep:
            return
        its = sorted((int(d[2:]), d) for d in os.listdir(self.save_path) if re.fullmatch(r"it\d+", d))
        import shutil

        for _, d in its[:-keep]:
            shutil.rmtree(os.path.join(self.save_path, d), ignore_errors=True)

    def save_ckpt(self, iteration: int, models, grad_manager, scheduler, dataloader, extra: dict, sync: bool = False,
                  sub_name: str | None = None, mark_latest: bool = True) -> str:
        self.join()
        path = self.iteration_dir(iteration, sub_name)
        if PM.world_rank == 0:
            os.makedirs(path, exist_ok=True)
        PM.barrier()
        os.makedirs(path, exist_ok=True)
        if getattr(grad_manager, "wait_param_gather", None):
            grad_manager.wait_param_gather()
        if torch.cuda.is_available():
            torch.cuda.synchronize()
            # a kernel that gave up a bounded wait (an unreduced gradient shard, an overfull expert buffer) left this
            # state inconsistent: fail here rather than mark such a checkpoint as the latest
            from ..ops import native

            native.raise_if_kernel_error()
        files = self.make_ckpt(models, grad_manager, scheduler, dataloader, extra)
        if getattr(self.cfg, "save_safetensors", False):
            from .hf_checkpoint import dump_safetensors

            dump_safetensors(models, os.path.join(path, "hf"), getattr(self.cfg, "model_config_path", None))
        if sync or not self.cfg.async_dump:
            self._write(files, path, mark_latest)
        else:
            def run():
                try:
                    self._write(files, path, mark_latest)
                except BaseException as e:  # surfaced by join()
                    self._error = e

            self._thread = threading.Thread(target=run, daemon=True)
            self._thread.start()
        return path

    @staticmethod
    def size_stat(file_objects: dict) -> str:
        """Log (rank 0) and return the tensor bytes per file of a checkpoint about to be written."""
        from .utils import size_report

        text = size_report(file_objects)
        if text:
            logger.info(text, at=0)
        return text

    def join_dumping_thread(self) -> None:
        """The reference's name for ``join``."""
        self.join()

    def join(self) -> None:
        if self._thread is not None:
            self._thread.join()
            self._thread = None
        if self._error is not None:
            err, self._error = self._error, None
            raise RuntimeError("asynchronous checkpoint write failed") from err

    # ------------------------------------------------------------------ load
    def load_ckpt(self, path: str, models, grad_manager, scheduler, dataloader) -> dict:
        """Restore what ``cfg.load_options`` selects; returns the ``extra`` dict.

        Model files exist only for DP rank 0 (EDP rank 0 for experts): those ranks read and the state
        is broadcast over the DP (EDP) group.  Optimizer shards are read by every rank."""
        opts = self.cfg.load_option
        layout = analyze_dir(path)
        here = {"tp": PM.size_of("TP"), "pp": PM.size_of("PP")}
        if (layout["tp"], layout["pp"]) != (here["tp"], here["pp"]):
            raise RuntimeError(f"checkpoint written with TP/PP {layout['tp']}/{layout['pp']}, running with "
                               f"{here['tp']}/{here['pp']}; convert through the HF safetensors export")
        src_name = f"TP{PM.rank_in('TP'):02d}_PP{PM.rank_in('PP'):03d}_DP000.pt"
        main = None
        mine = os.path.join(path, rank_file_name())
        reader = PM.rank_in("DP") == 0
        ep = PM.size_of("EP") > 1
        share = bool(getattr(self.cfg, "broadcast_from_dp0", True)) and PM.size_of("DP") > 1

        def load(file):
            return torch.load(file, map_location="cpu", weights_only=False)

        def model_part(state: dict, experts: bool) -> dict:
            """The model entries of a rank file, keeping expert tensors only (or everything else only)."""
            return {k: {n: t for n, t in sd.items() if (".experts." in n) == experts}
                    for k, sd in state.items() if k.startswith("model")}

        own = load(mine) if os.path.exists(mine) else {}
        # everything but expert weights is equal inside a DP group: the first replica's file holds it.  It reads and
        # broadcasts; with broadcast_from_dp0 off every rank reads that file itself (file-system traffic, no collective)
        first = own if reader else (None if share else load(os.path.join(path, src_name)))
        common = None
        if first is not None:
            common = {k: v for k, v in first.items() if k in ("extra", "scheduler")}
            common.update(model_part(first, experts=False) if ep else {k: v for k, v in first.items() if k.startswith("model")})
        if share:
            dev = "cuda" if torch.cuda.is_available() and PM.backend == "nccl" else "cpu"
            common = broadcast_tensors(common, src=PM.ranks_of("DP")[0], group=PM.group_of("DP"), device=dev)
        main = dict(common)
        if ep:
            # expert weights differ between the EP ranks of a DP group; they are equal inside an EDP group, whose first
            # rank wrote them into its own file
            experts = model_part(own, experts=True) if PM.rank_in("EDP") == 0 else None
            if PM.size_of("EDP") > 1:
                dev = "cuda" if torch.cuda.is_available() and PM.backend == "nccl" else "cpu"
                experts = broadcast_tensors(experts, src=PM.ranks_of("EDP")[0], group=PM.group_of("EDP"), device=dev)
            for k, sd in (experts or {}).items():
                main[k] = {**main.get(k, {}), **sd}
        if "rng_state" in own:
            main["rng_state"] = own["rng_state"]
        extra = main.get("extra", {})
        if opts.model:
            for i, m in enumerate(models):
                key = "model" if len(models) == 1 else f"model{i}"
                if key in main:
                    um = unwrap_model(m)
                    missing = um.load_state_dict(main[key], strict=False)
                    lost = [k for k in missing.missing_keys if not k.endswith("_extra_state")]
                    if lost and getattr(self.cfg, "strict_load_model", False):
                        raise RuntimeError(f"checkpoint {path} lacks {len(lost)} tensors of {key}: {lost[:5]} ...")
                    if lost:
                        logger.warning(f"missing keys when loading {key}: {lost[:5]} ...", at=None)
        opt_file = os.path.join(path, rank_file_name(opt=True))
        if not os.path.exists(opt_file):
            opt_file = os.path.join(path, src_name.replace(".pt", "_OPT.pt"))
        old_dp = optimizer_dp_size(path)
        sharded = bool(getattr(grad_manager, "shard_optimizer", False))
        if opts.optimizer and grad_manager is not None and sharded and old_dp not in (0, PM.size_of("DP")):
            # the shards on disk were cut for another data-parallel size
            if not getattr(self.cfg, "reshard_optimizer_state", False):
                raise RuntimeError(
                    f"checkpoint {path} holds optimizer shards of {old_dp} data-parallel ranks, this job has "
                    f"{PM.size_of('DP')}: set checkpoint_cfg.reshard_optimizer_state=True to re-cut them, or load "
                    f"without the optimizer (checkpoint_cfg.load_option.optimizer=False)")
            prefix = f"TP{PM.rank_in('TP'):02d}_PP{PM.rank_in('PP'):03d}_DP"
            grad_manager.load_resharded_state(
                lambda r: torch.load(os.path.join(path, f"{prefix}{r:03d}_OPT.pt"), map_location="cpu", weights_only=False),
                old_dp, strict=bool(getattr(self.cfg, "reshard_optimizer_strict", True)))
        elif opts.optimizer and grad_manager is not None and os.path.exists(opt_file):
            grad_manager.load_state_dict(torch.load(opt_file, map_location="cpu", weights_only=False))
        elif opts.model and grad_manager is not None and hasattr(grad_manager, "refresh_masters_from_params"):
            grad_manager.refresh_masters_from_params()
        if opts.scheduler and scheduler is not None and "scheduler" in main:
            scheduler.load_state_dict(main["scheduler"])
        data_file = os.path.join(path, "data.pkl")
        if opts.data and dataloader is not None and os.path.exists(data_file) and hasattr(dataloader, "load_state_dict"):
            with open(data_file, "rb") as f:
                dataloader.load_state_dict(pickle.load(f))
        if opts.rng_state and "rng_state" in main:
            try:
                PM.set_all_rng(main["rng_state"])
            except Exception as e:
                logger.warning(f"rng state not restored: {e}", at=None)
        return extra if isinstance(extra, dict) else {}
