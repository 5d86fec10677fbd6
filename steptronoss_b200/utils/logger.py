"""Rank-aware logging and the scalar writer (reference ``steptronoss/utils/logger.py:19-241``).

``logger.info(msg, at=0)`` prints only on the given global rank (``at=None``: every rank,
``at=-1``: last rank).  Built on loguru when present, on ``logging`` otherwise.
"""
from __future__ import annotations

import logging
import os


def _rank() -> int:
    return int(os.getenv("RANK", "0"))


def _world() -> int:
    return int(os.getenv("WORLD_SIZE", "1"))


class _RankLogger:
    def __init__(self):
        try:
            from loguru import logger as _lg

            self._lg, self._loguru = _lg, True
        except ImportError:  # pragma: no cover
            logging.basicConfig(level=logging.INFO, format="%(asctime)s %(levelname)s %(message)s")
            self._lg, self._loguru = logging.getLogger("stb200"), False

    def _emit(self, level: str, msg, at=0, **kw):
        if at is not None:
            target = at if at >= 0 else _world() + at
            if _rank() != target:
                return
        msg = str(msg)
        if self._loguru:
            self._lg.opt(depth=2).log(level.upper(), msg.replace("{", "{{").replace("}", "}}") if False else msg)
        else:
            getattr(self._lg, level)(msg)

    def info(self, msg, at=0, **kw):
        self._emit("info", msg, at)

    def warning(self, msg, at=None, **kw):
        self._emit("warning", msg, at)

    def error(self, msg, at=None, **kw):
        self._emit("error", msg, at)

    def debug(self, msg, at=0, **kw):
        self._emit("debug", msg, at)

    def success(self, msg, at=0, **kw):
        self._emit("success" if self._loguru else "info", msg, at)

    def exception(self, msg, at=None, **kw):
        self._emit("error", msg, at)

    def add(self, *a, **k):
        if self._loguru:
            return self._lg.add(*a, **k)

    def remove(self, *a, **k):
        if self._loguru:
            return self._lg.remove(*a, **k)


logger = _RankLogger()


def setup_logger(log_dir: str, per_rank_file: bool = True) -> None:
    """Add a per-rank log file under ``log_dir`` (created on demand)."""
    os.makedirs(log_dir, exist_ok=True)
    if per_rank_file:
        logger.add(os.path.join(log_dir, f"rank{_rank():04d}.log"), level="INFO", enqueue=False)


class StepWriter:
    """Scalar / histogram / text writer over TensorBoard and (optionally) wandb."""

    def __init__(self, log_dir: str, project_name=None, exp_name=None, backend=("tensorboard",), exp=None):
        self.writers = []
        self.log_dir = log_dir
        os.makedirs(log_dir, exist_ok=True)
        if "tensorboard" in backend:
            try:
                from torch.utils.tensorboard import SummaryWriter

                self.writers.append(SummaryWriter(log_dir=log_dir))
            except Exception as e:  # tensorboard not installed
                logger.warning(f"tensorboard writer unavailable: {e}", at=None)
        self._wandb = None
        if "wandb" in backend and os.getenv("WANDB_API_KEY"):
            try:
                import wandb

                entity, _, rest = (project_name or "").partition("/")
                proj, _, tag = rest.partition(":")
                self._wandb = wandb.init(project=proj or None, entity=entity or None, name=exp_name,
                                         tags=[tag] if tag else None, config=exp.to_dict(rep=True) if exp else None)
            except Exception as e:
                logger.warning(f"wandb writer unavailable: {e}", at=None)

    def add_scalar(self, key, value, global_step=None):
        for w in self.writers:
            w.add_scalar(key, value, global_step)
        if self._wandb is not None:
            self._wandb.log({key: value}, step=global_step)

    def add_histogram(self, key, values, global_step=None):
        for w in self.writers:
            w.add_histogram(key, values, global_step)

    def add_text(self, key, text, global_step=None):
        for w in self.writers:
            w.add_text(key, text, global_step)

    def flush(self):
        for w in self.writers:
            w.flush()

    def close(self):
        for w in self.writers:
            w.close()
        if self._wandb is not None:
            self._wandb.finish()
