"""MeshConnector on 4 gloo ranks: a TP=4 text mesh hands a batch to a DP=4 vision mesh and gets it back."""
import os

import torch
import torch.multiprocessing as mp

from tests.dist_helpers import free_port


def _worker(rank, world, port, q):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port))
    torch.set_num_threads(1)
    try:
        from steptronoss_b200.exp.base_exp import ParallelConfig
        from steptronoss_b200.models.common.mesh_connector import MeshConnector
        from steptronoss_b200.parallel.state import PM

        PM.initialize(backend="gloo")
        text, vision = ParallelConfig(), ParallelConfig()
        text.tensor_model_parallel_size = 2          # 2 replicas of TP=2 (both TP ranks hold the same batch)
        vision.context_parallel_size = 2             # 2 replicas of 2 nodes: the batch of a replica is split in two
        for c in (text, vision):
            c.expert_tensor_parallel_size = 1
        PM.set_mesh(text)
        conn = MeshConnector(text, vision, is_data_source=True, dup_dim=("TP",))
        replica = rank // 2
        batch = torch.arange(5 * 3, dtype=torch.float32).reshape(5, 3) + 100 * replica   # identical on both TP ranks
        shard = conn.forward(batch)
        feat = shard * 2 if shard is not None else None
        back = conn.backward(feat)
        q.put((rank, None if shard is None else shard.tolist(), None if back is None else back.tolist(), None))
        torch.distributed.barrier()
    except BaseException:
        import traceback

        q.put((rank, None, None, traceback.format_exc()))
        raise


def test_text_to_vision_and_back():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = free_port()
    procs = [ctx.Process(target=_worker, args=(r, 4, port, q)) for r in range(4)]
    for p in procs:
        p.start()
    res = {}
    try:
        for _ in range(4):
            rank, shard, back, err = q.get(timeout=120)
            assert err is None, err
            res[rank] = (shard, back)
    finally:
        for p in procs:
            p.join(timeout=30)
            if p.is_alive():
                p.kill()
    for rank, (shard, back) in res.items():
        replica = rank // 2
        full = (torch.arange(15, dtype=torch.float32).reshape(5, 3) + 100 * replica)
        assert back == (full * 2).tolist(), (rank, back)
    # under the vision mesh the two nodes of a replica get 3 and 2 rows of its 5-row batch
    assert [len(res[r][0]) for r in range(4)] == [3, 2, 3, 2]
    seen = sorted(tuple(r) for s, _ in res.values() for r in s)
    want = sorted(tuple(r) for rep in range(2) for r in (torch.arange(15, dtype=torch.float32).reshape(5, 3) + 100 * rep).tolist())
    assert seen == want
