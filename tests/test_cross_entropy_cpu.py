"""Vocab-parallel cross-entropy: against torch on one shard, label smoothing against its definition, and two
vocabulary shards on gloo ranks against the unsharded result."""
import os

import torch
import torch.multiprocessing as mp
import torch.nn.functional as F

from tests.dist_helpers import free_port


def test_matches_torch_and_reports_the_argmax():
    from steptronoss_b200.ops import vocab_parallel_cross_entropy

    torch.manual_seed(0)
    logits = torch.randn(9, 17, requires_grad=True)
    labels = torch.randint(0, 17, (9,))
    loss, pred = vocab_parallel_cross_entropy(logits, labels)
    assert torch.allclose(loss, F.cross_entropy(logits, labels, reduction="none"), atol=1e-6)
    assert torch.equal(pred, logits.argmax(-1))
    loss.mean().backward()
    g = logits.grad.clone()
    logits.grad = None
    F.cross_entropy(logits, labels).backward()
    assert torch.allclose(g, logits.grad, atol=1e-6)


def test_label_smoothing_follows_its_definition():
    from steptronoss_b200.ops import vocab_parallel_cross_entropy

    torch.manual_seed(1)
    K, a = 11, 0.1
    logits = torch.randn(5, K, dtype=torch.float64, requires_grad=True)
    labels = torch.randint(0, K, (5,))
    target = torch.full((5, K), a / (K - 1), dtype=torch.float64)       # a spread over the other K-1 classes
    target.scatter_(1, labels[:, None], 1.0 - a)
    want = -(target * F.log_softmax(logits, -1)).sum(-1)
    loss, _ = vocab_parallel_cross_entropy(logits.float(), labels, label_smoothing=a)
    assert torch.allclose(loss.double(), want, atol=1e-5)
    x = logits.detach().float().requires_grad_(True)
    vocab_parallel_cross_entropy(x, labels, label_smoothing=a)[0].sum().backward()
    want.sum().backward()
    assert torch.allclose(x.grad.double(), logits.grad, atol=1e-5)


def _worker(rank, world, port, q):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port))
    torch.set_num_threads(1)
    try:
        import torch.distributed as dist

        from steptronoss_b200.ops import vocab_parallel_cross_entropy

        dist.init_process_group("gloo", rank=rank, world_size=world)
        torch.manual_seed(2)
        full = torch.randn(6, 16)
        labels = torch.randint(0, 16, (6,))
        shard = full[:, rank * 8:(rank + 1) * 8].clone().requires_grad_(True)
        out = {}
        for a in (0.0, 0.2):
            shard.grad = None
            loss, pred = vocab_parallel_cross_entropy(shard, labels, rank * 8, dist.group.WORLD, label_smoothing=a)
            loss.sum().backward()
            out[a] = (loss.tolist(), pred.tolist(), shard.grad.tolist())
        q.put((rank, out, full.tolist(), labels.tolist(), None))
        dist.barrier()
    except BaseException:
        import traceback

        q.put((rank, None, None, None, traceback.format_exc()))
        raise


def test_two_vocabulary_shards_equal_the_whole():
    from steptronoss_b200.ops import vocab_parallel_cross_entropy

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = {}
    try:
        for _ in range(2):
            rank, out, full, labels, err = q.get(timeout=120)
            assert err is None, err
            res[rank] = out
    finally:
        for p in procs:
            p.join(timeout=30)
            if p.is_alive():
                p.kill()
    full, labels = torch.tensor(full), torch.tensor(labels)
    for a in (0.0, 0.2):
        x = full.clone().requires_grad_(True)
        loss, pred = vocab_parallel_cross_entropy(x, labels, label_smoothing=a)
        loss.sum().backward()
        for r in (0, 1):
            l, p, g = res[r][a]
            assert torch.allclose(torch.tensor(l), loss, atol=1e-5) and p == pred.tolist()
            assert torch.allclose(torch.tensor(g), x.grad[:, r * 8:(r + 1) * 8], atol=1e-5)
