"""Spawn gloo ranks on CPU that train the tiny experiment under a given parallel layout."""
from __future__ import annotations

import os
import socket

import torch
import torch.multiprocessing as mp


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _build(make_tiny_exp, exp_kwargs):
    exp_kwargs = dict(exp_kwargs)
    extra = exp_kwargs.pop("set", {})                      # dotted config paths to set after the experiment is built
    exp = make_tiny_exp(**exp_kwargs)
    for path, value in extra.items():
        node = exp
        *parents, leaf = path.split(".")
        for part in parents:
            node = getattr(node, part)
        setattr(node, leaf, value)
    return exp


def _worker(rank, world, port, exp_kwargs, steps, q):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port))
    torch.set_num_threads(1)
    try:
        from steptronoss_b200.parallel.state import PM
        from tests.tiny_exp import make_tiny_exp

        PM.initialize(backend="gloo")
        exp = _build(make_tiny_exp, exp_kwargs)
        exp.seed = 0
        tr = exp.trainer_cfg.get_trainer_cls()(exp=exp)
        tr.before_train()
        losses = []
        for _ in range(steps):
            tr.train_step()
            tr.iteration += 1
            tr.training_log()
            losses.append(tr.history[-1]["lm_loss"])
        norms = [tr.history[i]["grad_norm"] for i in range(steps)]
        parts = {k.split("/", 1)[1]: float(v) for k, v in tr.last_metrics.items() if k.startswith("grad_norms/")}
        if parts:                                           # detailed norms were asked for: hand them back with the norms
            norms = {"total": norms, "parts": parts}
        q.put((rank, losses, norms, None))
        torch.distributed.barrier()
    except BaseException as e:  # surface the failure to the parent instead of hanging it
        import traceback

        q.put((rank, None, None, traceback.format_exc()))
        raise


def run_ranks(world: int, exp_kwargs: dict, steps: int = 3, timeout: int = 300):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, exp_kwargs, steps, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = []
    try:
        for _ in range(world):
            item = q.get(timeout=timeout)
            if item[3] is not None:
                raise RuntimeError(f"rank {item[0]} failed:\n{item[3]}")
            results.append(item)
    finally:
        for p in procs:
            p.join(timeout=30)
            if p.is_alive():
                p.kill()
    return sorted(results, key=lambda t: t[0])


def run_single(exp_kwargs: dict, steps: int = 3):
    from tests.tiny_exp import make_tiny_exp

    os.environ.pop("WORLD_SIZE", None)
    exp = _build(make_tiny_exp, exp_kwargs)
    exp.seed = 0
    tr = exp.trainer_cfg.get_trainer_cls()(exp=exp)
    tr.before_train()
    losses = []
    for _ in range(steps):
        tr.train_step()
        tr.iteration += 1
        tr.training_log()
        losses.append(tr.history[-1]["lm_loss"])
    return losses, [h["grad_norm"] for h in tr.history]


def _call_worker(rank, world, port, fn, q):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port))
    torch.set_num_threads(1)
    try:
        from steptronoss_b200.parallel.state import PM

        PM.initialize(backend="gloo")
        q.put((rank, fn(rank, world), None))
        torch.distributed.barrier()
    except BaseException:
        import traceback

        q.put((rank, None, traceback.format_exc()))
        raise


def call_on_ranks(fn, world: int, timeout: int = 120) -> dict:
    """Run the module-level function ``fn(rank, world)`` on ``world`` gloo ranks; returns ``{rank: result}``."""
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = free_port()
    procs = [ctx.Process(target=_call_worker, args=(r, world, port, fn, q)) for r in range(world)]
    for p in procs:
        p.start()
    out = {}
    try:
        for _ in range(world):
            rank, res, err = q.get(timeout=timeout)
            if err is not None:
                raise RuntimeError(f"rank {rank} failed:\n{err}")
            out[rank] = res
    finally:
        for p in procs:
            p.join(timeout=30)
            if p.is_alive():
                p.kill()
    return out
