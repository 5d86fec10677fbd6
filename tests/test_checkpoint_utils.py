"""Checkpoint helpers: sizes, host copies, per-rank names, expert split, chunked byte broadcast."""
import numpy as np
import pytest
import torch

from steptronoss_b200.checkpointing import utils as cu
from steptronoss_b200.checkpointing.local_checkpoint import Checkpointer
from steptronoss_b200.exp.base_exp import ParallelConfig


def test_sizes_and_host_copies():
    state = {"a": torch.zeros(4, 8, dtype=torch.bfloat16), "b": [np.zeros(3, dtype=np.float64), {"c": torch.ones(2)}],
             "step": 7, "name": "x"}
    assert cu.recur_stat(state) == 64 + 24 + 8
    assert cu.size_report({"model.pt": state, "meta": {"it": 1}}) == "model.pt: 0.0 G | meta: NOTENSOR"
    assert Checkpointer.size_stat({"meta": {"it": 1}}) == "meta: NOTENSOR"
    copy = cu.move_to_memory(state)
    assert copy["a"].data_ptr() != state["a"].data_ptr() and torch.equal(copy["b"][1]["c"], state["b"][1]["c"])
    copy["b"][0][0] = 5.0
    assert state["b"][0][0] == 0.0 and copy["step"] == 7                  # arrays and leaves are copies too
    t = torch.arange(3.0)
    assert cu.move_tensor_to_memory(t).data_ptr() != t.data_ptr()


def test_expert_split_keeps_shared_entries_on_both_sides():
    sd = {"iteration": 3, "model0": {"layers.0.attn.wqkv": 1, "layers.1.moe.experts.w1": 2},
          "model1": {"layers.2.moe.experts.w2": 3, "norm.weight": 4}}
    experts, rest = cu.split_state_dict(sd)
    assert experts == {"iteration": 3, "model0": {"layers.1.moe.experts.w1": 2}, "model1": {"layers.2.moe.experts.w2": 3}}
    assert rest == {"iteration": 3, "model0": {"layers.0.attn.wqkv": 1}, "model1": {"norm.weight": 4}}
    assert cu.split_state_dict({"iteration": 1}) == ({"iteration": 1}, {"iteration": 1})


def _names_worker(rank, world):
    import os
    import tempfile

    from steptronoss_b200.parallel.state import PM

    pc = ParallelConfig()
    pc.tensor_model_parallel_size = 2
    PM.set_mesh(pc)
    name = cu.get_rank_specific_name()
    d = tempfile.mkdtemp()
    for f in ("TP00_PP000_DP000.pt", "TP01_PP000_DP000.pt"):
        open(os.path.join(d, f), "w").close()
    mine = os.path.basename(cu.find_rank_specific_path(d))
    open(os.path.join(d, "TP02_PP000_DP000.pt"), "w").close()            # a directory written with TP = 3
    try:
        cu.find_rank_specific_path(d)
        mismatch = False
    except AssertionError:
        mismatch = True
    blob = bytes(range(256)) * 10 if rank == 0 else None
    got = cu.chunked_broadcast_bytes(blob, src=0, chunk_size=1000)
    return name, mine, mismatch, len(got), got[:4] == bytes([0, 1, 2, 3]) and got[-1] == 255


def test_rank_names_and_chunked_broadcast_on_two_ranks():
    from tests.dist_helpers import call_on_ranks

    got = call_on_ranks(_names_worker, 2)
    assert got[0][:3] == ("TP00_PP000_DP000", "TP00_PP000_DP000.pt", True)
    assert got[1][:3] == ("TP01_PP000_DP000", "TP01_PP000_DP000.pt", True)
    assert got[0][3:] == got[1][3:] == (2560, True)
