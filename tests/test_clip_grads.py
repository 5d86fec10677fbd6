"""Clipping and zero counting over plain parameter lists: one process and two gloo ranks of tensor parallelism."""
import pytest
import torch

from steptronoss_b200.exp.base_exp import ParallelConfig
from steptronoss_b200.optim.clip_grads import clip_grad_norm_fp32, count_zeros_fp32


def _params():
    a, b = torch.nn.Parameter(torch.zeros(3)), torch.nn.Parameter(torch.zeros(2, 2))
    a.grad, b.grad = torch.tensor([3.0, 0.0, 4.0]), torch.tensor([[0.0, 12.0], [0.0, 0.0]])
    return a, b


def test_clip_and_count_on_one_process():
    a, b = _params()
    assert count_zeros_fp32([a, b]) == 4.0
    norm = clip_grad_norm_fp32([a, b], [a.grad, b.grad], max_norm=6.5)
    assert norm == pytest.approx(13.0)                                   # sqrt(9 + 16 + 144)
    assert torch.allclose(a.grad, torch.tensor([1.5, 0.0, 2.0]), atol=1e-5) and float(b.grad[0, 1]) == pytest.approx(6.0, abs=1e-5)
    assert clip_grad_norm_fp32([a, b], [a.grad, b.grad], max_norm=100.0) == pytest.approx(6.5, abs=1e-4)
    assert float(a.grad[0]) == pytest.approx(1.5, abs=1e-5)              # below the limit: untouched
    assert clip_grad_norm_fp32(a, a.grad, 1.0, norm_type=float("inf")) == pytest.approx(2.0, abs=1e-5)
    b.shared = True
    assert count_zeros_fp32([a, b]) == 1.0
    assert count_zeros_fp32([torch.nn.Parameter(torch.zeros(1))]) == 0.0 # no gradient at all


def _two_rank_worker(rank, world):
    from steptronoss_b200.parallel.state import PM

    pc = ParallelConfig()
    pc.tensor_model_parallel_size = 2
    PM.set_mesh(pc)
    sharded, replicated = torch.nn.Parameter(torch.zeros(2)), torch.nn.Parameter(torch.zeros(2))
    sharded.tensor_model_parallel = True
    sharded.grad = torch.tensor([3.0, 0.0]) if rank == 0 else torch.tensor([0.0, 4.0])
    replicated.grad = torch.tensor([12.0, 0.0])
    counted = [sharded.grad] + ([replicated.grad] if rank == 0 else [])
    zeros = count_zeros_fp32([sharded, replicated], PM.group_of("TP"))
    norm = clip_grad_norm_fp32([sharded, replicated], counted, 1.3, model_parallel_group=PM.group_of("TP"))
    return zeros, norm, sharded.grad.tolist(), replicated.grad.tolist()


def test_replicated_gradients_count_once_over_two_ranks():
    from tests.dist_helpers import call_on_ranks

    got = call_on_ranks(_two_rank_worker, 2)
    for rank in (0, 1):
        zeros, norm, _, rep = got[rank]
        assert zeros == 3.0 and norm == pytest.approx(13.0)              # 1 + 1 zeros of the shards, 1 of the replica
        assert rep[0] == pytest.approx(1.2, abs=1e-5)                    # every copy is scaled
    assert got[0][2][0] == pytest.approx(0.3, abs=1e-5) and got[1][2][1] == pytest.approx(0.4, abs=1e-5)
