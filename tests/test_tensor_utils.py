"""Partition and viewless-tensor helpers of the tensor-parallel layer: one process, and two gloo ranks for the
gather of flat shards."""
import pytest
import torch

from steptronoss_b200.exp.base_exp import ParallelConfig

from steptronoss_b200.parallel import tensor_utils as tu


def test_divide_and_vocab_ranges():
    assert tu.divide(12, 4) == 3
    with pytest.raises(AssertionError):
        tu.divide(10, 4)
    assert tu.VocabUtility.vocab_range_from_global_vocab_size(1024, 3, 4) == (768, 1024)
    assert tu.VocabUtility.vocab_range_from_per_partition_vocab_size(100, 2, 8) == (200, 300)


def test_split_along_last_dim():
    x = torch.arange(24).view(2, 12)
    a, b, c = tu.split_tensor_along_last_dim(x, 3)
    assert torch.equal(b, x[:, 4:8]) and b._base is not None
    parts = tu.split_tensor_along_last_dim(x, 3, contiguous_split_chunks=True)
    assert all(p.is_contiguous() for p in parts)
    with pytest.raises(AssertionError):
        tu.split_tensor_along_last_dim(x, 5)


def test_flat_shards_on_one_rank_round_trip():
    x = torch.arange(10.0).view(2, 5)
    piece = tu.split_tensor_into_1d_equal_chunks(x)
    assert piece.data_ptr() == x.data_ptr() and piece.shape == (10,)
    copy = tu.split_tensor_into_1d_equal_chunks(x, new_buffer=True)
    assert copy.data_ptr() != x.data_ptr()
    assert torch.equal(tu.gather_split_1d_tensor(piece), x.reshape(-1))


def test_viewless_tensor_drops_the_base_but_keeps_the_graph():
    base = torch.randn(4, 6, requires_grad=True)
    view = (base * 2)[1:3]
    assert view._base is not None
    with pytest.raises(AssertionError):
        tu.assert_viewless_tensor(view)
    out = tu.make_viewless_tensor(view, requires_grad=True, keep_graph=True)
    assert out._base is None and out.data_ptr() == view.data_ptr() and tu.assert_viewless_tensor([out]) == [out]
    out.sum().backward()
    assert torch.equal(base.grad[1:3], torch.full((2, 6), 2.0)) and float(base.grad[0].abs().sum()) == 0.0
    detached = tu.make_viewless_tensor(view.detach(), requires_grad=False, keep_graph=False)
    assert detached._base is None and not detached.requires_grad
    plain = torch.zeros(3)
    assert tu.make_viewless_tensor(plain, False, False) is plain
    tu.safely_set_viewless_tensor_data(detached, torch.ones(2))
    assert detached.shape == (2,)
    with pytest.raises(AssertionError):
        tu.safely_set_viewless_tensor_data(view, torch.ones(2))


def test_which_parameter_copy_counts():
    p = torch.nn.Parameter(torch.zeros(2))
    assert tu.param_is_not_shared(p) and tu.param_is_not_tensor_parallel_duplicate(p)     # one rank: TP rank 0
    p.shared = True
    p.tensor_model_parallel = True
    assert not tu.param_is_not_shared(p) and tu.param_is_not_tensor_parallel_duplicate(p)
    assert tu.param_is_not_expert_parallel_duplicate(p)


def _flat_shards_worker(rank, world):
    from steptronoss_b200.parallel.state import PM

    pc = ParallelConfig()
    pc.tensor_model_parallel_size = 2
    PM.set_mesh(pc)
    full = torch.arange(12.0).view(3, 4)
    mine = tu.split_tensor_into_1d_equal_chunks(full)
    return {"piece": mine.tolist(), "gathered": tu.gather_split_1d_tensor(mine).tolist(),
            "counts": tu.param_is_not_tensor_parallel_duplicate(torch.nn.Parameter(torch.zeros(1)))}


def test_flat_shards_gather_over_two_ranks():
    from tests.dist_helpers import call_on_ranks

    got = call_on_ranks(_flat_shards_worker, 2)
    assert got[0]["piece"] == list(range(6)) and got[1]["piece"] == list(range(6, 12))
    assert got[0]["gathered"] == got[1]["gathered"] == [float(i) for i in range(12)]
    assert got[0]["counts"] and not got[1]["counts"]                      # a replicated parameter counts once


def _padded_split_worker(rank, world):
    from steptronoss_b200.parallel import mappings
    from steptronoss_b200.parallel.state import PM

    pc = ParallelConfig()
    pc.tensor_model_parallel_size = 2
    PM.set_mesh(pc)
    x = torch.arange(14.0).view(7, 2)
    share, pad = mappings.split_along_first_dim_with_padding(x)
    even, pad0 = mappings.split_along_first_dim_with_padding(x[:6])
    sliced = mappings.slice_to_sequence_parallel_region(x[:6].clone().requires_grad_())
    try:
        mappings.split_along_first_dim_with_padding(x[:1])
        few = False
    except AssertionError:
        few = True
    return tuple(share.shape), pad, share[:3].tolist(), tuple(even.shape), pad0, sliced.tolist(), few


def test_first_dim_split_with_padding_over_two_ranks():
    from steptronoss_b200.parallel import mappings
    from tests.dist_helpers import call_on_ranks

    x = torch.zeros(5, 2)
    assert mappings.split_along_first_dim_with_padding(x) is x                 # a group of one: untouched
    got = call_on_ranks(_padded_split_worker, 2)
    assert got[0][:3] == ((4, 2), 1, [[0.0, 1.0], [2.0, 3.0], [4.0, 5.0]])
    assert got[1][:3] == ((4, 2), 1, [[8.0, 9.0], [10.0, 11.0], [12.0, 13.0]])  # three real rows and one of padding
    assert got[0][3:5] == got[1][3:5] == ((3, 2), 0)
    assert got[0][5] == [[0.0, 1.0], [2.0, 3.0], [4.0, 5.0]] and got[1][5] == [[6.0, 7.0], [8.0, 9.0], [10.0, 11.0]]
    assert got[0][6] and got[1][6]


def test_model_wrapper_base_and_precision_helpers():
    from steptronoss_b200.models.module import (ModelWrapperBase, conversion_helper, float16_to_fp32, fp32_to_float16,
                                                unwrap_model)

    inner = torch.nn.Linear(3, 2)
    wrapped = ModelWrapperBase(ModelWrapperBase(inner))
    assert unwrap_model(wrapped) is inner and set(wrapped.state_dict()) == {"weight", "bias"}
    wrapped.load_state_dict({"weight": torch.ones(2, 3), "bias": torch.zeros(2)})
    assert torch.equal(wrapped(torch.ones(1, 3)), torch.full((1, 2), 3.0))
    nest = (torch.ones(2), [torch.ones(2, dtype=torch.int64), "text"], None)
    low = fp32_to_float16(nest)
    assert isinstance(low, tuple) and low[0].dtype == torch.bfloat16 and low[1][0].dtype == torch.int64 and low[1][1] == "text"
    assert float16_to_fp32(low)[0].dtype == torch.float32 and fp32_to_float16(nest, torch.float16)[0].dtype == torch.float16
    assert conversion_helper([1, (2, 3)], lambda v: v * 2) == [2, (4, 6)]


def _p2p_worker(rank, world):
    from types import SimpleNamespace

    from steptronoss_b200.parallel.pipeline import p2p
    from steptronoss_b200.parallel.state import PM

    pc = ParallelConfig()
    pc.pipeline_model_parallel_size = 2
    PM.set_mesh(pc)
    cfg = SimpleNamespace(params_dtype=torch.float32, variable_seq_lengths=False)
    shape = (3, 2)
    if rank == 0:
        assert p2p.recv_forward(cfg, shape) is None                       # the first stage receives nothing
        p2p.send_forward(cfg, torch.full(shape, 7.0), shape)
        grad = p2p.recv_backward(cfg, shape)
        p2p.send_backward(cfg, grad, shape)                               # no previous stage: nothing happens
        back = p2p.send_forward_recv_backward(cfg, torch.full(shape, 9.0), shape)
        return grad.tolist(), back.tolist()
    act = p2p.recv_forward(cfg, shape)
    p2p.send_forward(cfg, act, shape)                                     # the last stage sends nothing
    p2p.send_backward(cfg, act * 2, shape)
    assert p2p.recv_backward(cfg, shape) is None
    again = p2p.send_backward_recv_forward(cfg, torch.full(shape, -1.0), shape)
    return act.tolist(), again.tolist()


def test_p2p_free_functions_over_two_stages():
    from tests.dist_helpers import call_on_ranks

    got = call_on_ranks(_p2p_worker, 2)
    assert got[1][0] == [[7.0, 7.0]] * 3 and got[0][0] == [[14.0, 14.0]] * 3
    assert got[1][1] == [[9.0, 9.0]] * 3 and got[0][1] == [[-1.0, -1.0]] * 3
