"""Keep copies of the token embedding that live on different pipeline stages identical.

A model whose later stage needs the input embedding again (a multi-token-prediction head embeds the next tokens on
the last stage) holds a second copy of the table there.  The copies start equal and must stay equal: their
gradients have to be summed before the optimizer step.  This module finds the holders, builds the process-group
family ``EMB_SYNC`` and performs the initial broadcast; the model does the per-step gradient sum on that family.

A model chunk takes part by setting ``need_mtp_sync = True`` and offering ``shared_embedding_parameters()`` (the
parameters to keep equal, same order on every holder).  Same role as the reference's ``mtp_initialize``
(``steptronoss/initialize.py:13-47``), which builds ``EMB_SYNC`` from an all-gather over the PP group.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..models.module import unwrap_model
from ..utils.logger import logger
from .state import PM

FAMILY = "EMB_SYNC"


def embedding_sync_rows(pp_rows: list, holder_stages: list) -> list:
    """Rows of the ``EMB_SYNC`` family: in every pipeline row the holder stages form one row; every other rank gets
    a row of its own kind (the stages that hold nothing), so that each rank of the world is in exactly one row."""
    held = sorted(set(holder_stages))
    rest = [i for i in range(len(pp_rows[0])) if i not in held]
    rows = [[row[i] for i in held] for row in pp_rows] if held else []
    if rest:
        rows += [[row[i] for i in rest] for row in pp_rows]
    return rows


def sync_shared_embeddings(models) -> list:
    """Build ``EMB_SYNC`` and make every holder's copy equal to the first stage's.  Returns this rank's row.

    Collective over the world: every rank calls it, holders or not."""
    holders = [m for m in models if getattr(unwrap_model(m), "need_mtp_sync", False)]
    if len(holders) > 1:
        raise AssertionError("at most one model chunk per rank may hold a shared embedding")
    pp = PM.size_of("PP")
    if not dist.is_initialized() or pp == 1:
        return [PM.world_rank]
    dev = next(unwrap_model(models[0]).parameters()).device if models else torch.device("cpu")
    mine = torch.tensor([1 if holders else 0], dtype=torch.int64, device=dev)
    every = torch.zeros(pp, dtype=torch.int64, device=dev)
    dist.all_gather_into_tensor(every, mine, group=PM.group_of("PP"))
    stages = [i for i, h in enumerate(every.tolist()) if h]
    # every pipeline row has the same holder stages (the layer map does not depend on the data/tensor coordinates)
    fam = PM.new_parallel(FAMILY, embedding_sync_rows(PM.world_ranks_of("PP"), stages))
    if holders and len(stages) > 1:
        row = PM.ranks_of(FAMILY)
        group = PM.group_of(FAMILY)
        for p in unwrap_model(holders[0]).shared_embedding_parameters():
            dist.broadcast(p.data, src=row[0], group=group)
    PM.barrier()
    logger.info(f"shared input embeddings synchronised over stages {stages}", at=0)
    return fam.ranks[fam.my_row]


def reduce_shared_embedding_grads(model) -> None:
    """Sum the gradients (``main_grad`` when the parameter has one) of the shared copies over ``EMB_SYNC``: call
    between backward and the optimizer step on every holder."""
    group = PM.group_of(FAMILY) if PM.has(FAMILY) else None
    if group is None:
        return
    for p in unwrap_model(model).shared_embedding_parameters():
        g = getattr(p, "main_grad", None)
        g = p.grad if g is None else g
        if g is not None:
            dist.all_reduce(g, group=group)
