"""Activation recomputation: plain checkpoint, the sanity check, and the variant that also frees the output."""
import pytest
import torch


def _mlp():
    torch.manual_seed(0)
    return torch.nn.Sequential(torch.nn.Linear(8, 16), torch.nn.GELU(), torch.nn.Dropout(0.5), torch.nn.Linear(16, 8))


def test_checkpoint_gives_the_same_gradients_under_dropout(monkeypatch):
    from steptronoss_b200.parallel.random import checkpoint

    net = _mlp()
    x = torch.randn(4, 8, requires_grad=True)
    torch.manual_seed(7)
    net(x).square().sum().backward()
    want = [p.grad.clone() for p in net.parameters()] + [x.grad.clone()]
    for p in net.parameters():
        p.grad = None
    x.grad = None
    monkeypatch.setenv("RECOMPUTE_SANITY_CHECK", "1")              # the recomputed output is compared with the first one
    torch.manual_seed(7)
    checkpoint(net, x).square().sum().backward()
    got = [p.grad for p in net.parameters()] + [x.grad]
    for a, b in zip(want, got):
        assert torch.allclose(a, b, atol=1e-6)


def test_output_is_released_and_refilled_before_the_consumer_needs_it():
    from steptronoss_b200.parallel.random import CheckpointWithoutOutput

    net, head = _mlp(), torch.nn.Linear(8, 3)
    x = torch.randn(4, 8, requires_grad=True)
    torch.manual_seed(11)
    head(net(x)).square().sum().backward()
    want = [p.grad.clone() for p in list(net.parameters()) + list(head.parameters())] + [x.grad.clone()]
    for p in list(net.parameters()) + list(head.parameters()):
        p.grad = None
    x.grad = None

    ck = CheckpointWithoutOutput()
    torch.manual_seed(11)
    h = ck.checkpoint(net, x)
    y = head(h)                                                    # the linear layer saved h for its weight gradient
    ck.discard_output_and_register_recompute(y)
    assert h.untyped_storage().size() == 0                         # nothing of h is held between forward and backward
    y.square().sum().backward()
    got = [p.grad for p in list(net.parameters()) + list(head.parameters())] + [x.grad]
    for a, b in zip(want, got):
        assert torch.allclose(a, b, atol=1e-6)
    assert h.untyped_storage().size() > 0


def test_backward_without_the_hook_says_what_is_missing():
    from steptronoss_b200.parallel.random import CheckpointWithoutOutput

    net = _mlp()
    x = torch.randn(2, 8, requires_grad=True)
    h = CheckpointWithoutOutput().checkpoint(net, x)
    with pytest.raises(RuntimeError, match="never recomputed"):
        h.sum().backward()


def _tp_worker(rank, world, port, q):
    import os

    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port))
    torch.set_num_threads(1)
    try:
        from steptronoss_b200.exp.base_exp import ParallelConfig
        from steptronoss_b200.parallel.random import checkpoint
        from steptronoss_b200.parallel.state import PM

        PM.initialize(backend="gloo")
        cfg = ParallelConfig()
        cfg.tensor_model_parallel_size, cfg.expert_tensor_parallel_size = 2, 1
        PM.set_mesh(cfg)
        torch.manual_seed(0)                                        # the same input on both ranks, as without SP
        x = torch.randn(6, 4, requires_grad=True)
        w = torch.randn(4, 4, requires_grad=True)
        y = checkpoint(lambda t, m: torch.tanh(t @ m), x, w, distribute_saved_activations=True)
        kept = [t.numel() for t in y.grad_fn.saved_tensors]
        y.square().sum().backward()
        gx, gw = x.grad.clone(), w.grad.clone()
        x.grad = w.grad = None
        torch.tanh(x @ w).square().sum().backward()
        q.put((rank, kept, bool(torch.allclose(gx, x.grad, atol=1e-6) and torch.allclose(gw, w.grad, atol=1e-6)), None))
        torch.distributed.barrier()
    except BaseException:
        import traceback

        q.put((rank, None, None, traceback.format_exc()))
        raise


def test_saved_input_is_split_over_the_tp_ranks_and_gathered_in_backward():
    import torch.multiprocessing as mp

    from tests.dist_helpers import free_port

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = free_port()
    procs = [ctx.Process(target=_tp_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    try:
        for _ in range(2):
            rank, kept, same, err = q.get(timeout=120)
            assert err is None, err
            assert kept == [12, 16] and same                        # half of the 24 input values, the whole weight
    finally:
        for p in procs:
            p.join(timeout=30)
            if p.is_alive():
                p.kill()
