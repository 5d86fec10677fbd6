"""Shared token-embedding copies on two pipeline stages: family rows, first broadcast, gradient sum (4 gloo ranks)."""
import os

import torch
import torch.multiprocessing as mp

from tests.dist_helpers import free_port


def test_rows_cover_every_rank_once():
    from steptronoss_b200.parallel.embedding_sync import embedding_sync_rows

    pp_rows = [[0, 2, 4, 6], [1, 3, 5, 7]]                     # two pipelines of four stages
    rows = embedding_sync_rows(pp_rows, [0, 3])
    assert rows == [[0, 6], [1, 7], [2, 4], [3, 5]]
    assert sorted(r for row in rows for r in row) == list(range(8))
    assert embedding_sync_rows(pp_rows, []) == pp_rows
    assert embedding_sync_rows(pp_rows, [0, 1, 2, 3]) == pp_rows


def _worker(rank, world, port, q):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port))
    torch.set_num_threads(1)
    try:
        from steptronoss_b200.exp.base_exp import ParallelConfig
        from steptronoss_b200.models.module import MegatronModule
        from steptronoss_b200.parallel import embedding_sync as es
        from steptronoss_b200.parallel.state import PM

        PM.initialize(backend="gloo")
        cfg = ParallelConfig()
        cfg.pipeline_model_parallel_size = 2
        cfg.expert_tensor_parallel_size = 1
        PM.set_mesh(cfg)

        class Stage(MegatronModule):
            need_mtp_sync = True

            def __init__(self):
                super().__init__()
                torch.manual_seed(100 + rank)                     # every copy starts different
                self.emb = torch.nn.Parameter(torch.randn(6, 4))

            def shared_embedding_parameters(self):
                return [self.emb]

        m = Stage()
        before = m.emb.detach().clone()
        row = es.sync_shared_embeddings([m])
        m.emb.main_grad = torch.full((6, 4), float(rank + 1))
        es.reduce_shared_embedding_grads(m)
        q.put((rank, row, PM.rank_in("PP"), before.tolist(), m.emb.detach().tolist(), float(m.emb.main_grad[0, 0]), None))
        torch.distributed.barrier()
    except BaseException:
        import traceback

        q.put((rank, None, None, None, None, None, traceback.format_exc()))
        raise


def test_copies_follow_the_first_stage_and_gradients_are_summed():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = free_port()
    procs = [ctx.Process(target=_worker, args=(r, 4, port, q)) for r in range(4)]
    for p in procs:
        p.start()
    res = {}
    try:
        for _ in range(4):
            rank, row, stage, before, after, grad, err = q.get(timeout=120)
            assert err is None, err
            res[rank] = (row, stage, before, after, grad)
    finally:
        for p in procs:
            p.join(timeout=30)
            if p.is_alive():
                p.kill()
    for rank, (row, stage, before, after, grad) in res.items():
        assert rank in row and len(row) == 2
        first = next(r for r in row if res[r][1] == 0)            # the first-stage member of this rank's row
        assert after == res[first][2]                             # everyone now holds the first stage's initial table
        assert grad == sum(r + 1 for r in row)
