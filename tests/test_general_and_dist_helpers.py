"""List / tensor helpers of ``utils.general`` and the object collectives of ``utils.dist_utils`` (2 gloo ranks)."""
import os
import random

import pytest
import torch
import torch.multiprocessing as mp

from tests.dist_helpers import free_port


def test_shifts_cumulative_lengths_and_splits():
    from steptronoss_b200.utils import general as g

    t = torch.tensor([1, 2, 3, 4])
    assert g.shift_left(t, pad=9).tolist() == [2, 3, 4, 9] and g.shift_right(t, pad=9, shift=2).tolist() == [9, 9, 1, 2]
    cu = g.lens_to_cum_len([3, 2, 4])
    assert cu.dtype == torch.int32 and cu.tolist() == [0, 3, 5, 9]
    assert g.get_position_id_from_cu_seqlens(cu).tolist() == [0, 1, 2, 0, 1, 0, 1, 2, 3]
    assert g.list_split(list(range(5)), 2) == [[0, 1, 2], [3, 4]] and g.list_split_T(list(range(5)), 2) == [[0, 2, 4], [1, 3]]
    assert g.list_chunk(list(range(5)), 2) == [[0, 1], [2, 3], [4]]
    parts = g.balanced_list_split(list("abcdef"), [9, 1, 1, 1, 1, 5], 2)
    assert sorted(x for p in parts for x in p) == list("abcdef")
    loads = [sum({"a": 9, "b": 1, "c": 1, "d": 1, "e": 1, "f": 5}[x] for x in p) for p in parts]
    assert sorted(loads) == [9, 9]
    even = g.balanced_list_split(list(range(6)), [5, 1, 1, 1, 1, 1], 2, number_balance=True)
    assert sorted(len(p) for p in even) == [3, 3]
    runs = g.balanced_list_split_keep_order(list(range(6)), [4, 1, 1, 4, 1, 1], 2)
    assert runs == [[0, 1, 2], [3, 4, 5]]
    assert g.balanced_list_split_keep_order([1, 2], [1, 1], 4) == [[1], [2], [], []]


def test_fork_rng_state_and_tensor_identity_cache():
    from steptronoss_b200.utils import general as g

    random.seed(5)
    torch.manual_seed(5)
    a = (random.random(), float(torch.rand(1)))
    random.seed(5)
    torch.manual_seed(5)
    with g.fork_rng_state(11):
        inside1 = float(torch.rand(1))
    b = (random.random(), float(torch.rand(1)))
    with g.fork_rng_state(11):
        inside2 = float(torch.rand(1))
    assert a == b and inside1 == inside2                      # the block neither disturbs nor depends on the outer streams

    calls = []

    @g.cache_with_tensor([True, False])
    def f(t, k):
        calls.append(k)
        return t.sum() * k

    x = torch.ones(3)
    assert float(f(x, 2)) == 6.0 and float(f(x, 2)) == 6.0 and calls == [2]
    assert float(f(x, 3)) == 9.0 and calls == [2, 3]
    x.add_(1)                                                 # same object, new version: not a hit
    assert float(f(x, 2)) == 12.0 and calls == [2, 3, 2]
    y = torch.ones(3)
    f(y, 2)
    assert calls == [2, 3, 2, 2]                              # equal values, another tensor: not a hit


def test_pickled_tensors_and_tp_resharding():
    from steptronoss_b200.utils import dist_utils as du

    obj = {"a": torch.arange(4), "b": ["x", 3.5, torch.ones(2, 2)]}
    back = du.tensor_to_dict(du.dict_to_tensor(obj))
    assert back["b"][:2] == ["x", 3.5] and torch.equal(back["a"], obj["a"]) and torch.equal(back["b"][2], obj["b"][2])
    full = torch.arange(24).reshape(4, 6)
    shards = du.redistributed_tp(list(full.chunk(2, dim=1)), dim=1, new_tp=3)
    assert len(shards) == 3 and torch.equal(torch.cat(shards, dim=1), full) and shards[0].shape == (4, 2)
    assert du.balanced_map(lambda v: v * v, [1, 2, 3]) == [1, 4, 9]           # one process: plain map
    assert du.replicated_map(lambda v: v * v, [1, 2, 3]) == [1, 4, 9]
    names = ["input", "ids", "n", "absent", "flag"]
    table, payload = du.pack_tensors({"input": torch.arange(6.0).reshape(6, 1), "ids": torch.arange(5, dtype=torch.int32),
                                      "n": 7, "absent": None, "flag": torch.tensor([True, False])}, names)
    back = du.unpack_tensors(table, payload, names)
    assert back["input"].shape == (6, 1) and back["ids"].dtype == torch.int32 and back["ids"].tolist() == [0, 1, 2, 3, 4]
    assert back["n"].tolist() == [7] and back["absent"] is None and back["flag"].tolist() == [True, False]
    assert du.concat_list_in_group([1, 2]) == [1, 2] and du.gather_object(["a"]) == [["a"]]
    assert du.all_to_all_objects(["only"]) == ["only"] and du.gather_dict({"k": 1}) == [{"k": 1}]


def _worker(rank, world, port, q):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port))
    torch.set_num_threads(1)
    try:
        import torch.distributed as dist

        from steptronoss_b200.utils import dist_utils as du

        dist.init_process_group("gloo", rank=rank, world_size=world)
        out = {}
        out["a2a"] = du.all_to_all_objects([f"{rank}->{d}" for d in range(world)])
        out["gathered"] = [d["r"] for d in du.all_gather_dict({"r": rank, "t": torch.full((2,), float(rank))})]
        g = du.gather_dict({"r": rank}, dst=1)
        out["gather_dst1"] = None if g is None else [d["r"] for d in g]
        if rank == 0:
            du.send_tensors({"w": torch.arange(3.0), "meta": ("m", [torch.ones(2, dtype=torch.int64)])}, dst=1)
        else:
            got = du.recv_tensors(src=0)
            out["recv"] = (got["w"].tolist(), got["meta"][0], got["meta"][1][0].tolist(), str(got["meta"][1][0].dtype))
        seen = []

        def work(v):
            seen.append(v)
            return v * 10

        out["map"] = du.replicated_map(work, [1, 2, 3, 4, 5], sizes=[5, 1, 1, 1, 1])
        out["did"] = sorted(seen)
        # per-rank lists of unequal length: evened out, mapped, results back at their owners
        mine = [0, 1, 2, 3, 4] if rank == 0 else [5]
        bal, info = du.list_balance(mine)
        out["balanced"] = bal
        out["restored"] = du.list_unbalance(bal, info)
        out["bmap"] = du.balanced_map(lambda v: v + 100, mine)
        out["concat"] = du.concat_list_in_group([rank, rank])
        out["concat_one"] = du.concat_list_in_group([torch.arange(3)] if rank == 1 else [])[0].tolist()
        out["gather_obj"] = du.gather_object([f"from{rank}"], dst=1)
        got = du.all_to_all_tensors([torch.full((rank + 1, d + 1), float(rank * 10 + d)) for d in range(world)])
        out["a2a_tensors"] = [(tuple(t.shape), float(t[0, 0])) for t in got]
        if rank == 0:
            du.send_obj({"k": [1, 2, torch.ones(2)]}, dst=1)
            du.wait_all(du.isend_packed_tensors({"input": torch.ones(3, 1), "pos": torch.arange(3), "none": None}, dst=1))
        else:
            o = du.recv_obj(src=0)
            out["recv_obj"] = (o["k"][:2], o["k"][2].tolist())
            t = du.recv_packed_tensors(["input", "pos", "none"], src=0)
            out["recv_packed"] = (tuple(t["input"].shape), t["pos"].tolist(), t["none"])
        b = du.broadcast_tensors({"x": torch.arange(4) + 1, "s": "hello"} if rank == 0 else None, src_rank=0)
        out["bcast"] = (b["x"].tolist(), b["s"])
        q.put((rank, out, None))
        dist.barrier()
    except BaseException:
        import traceback

        q.put((rank, None, traceback.format_exc()))
        raise


def test_object_collectives_on_two_ranks():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = {}
    try:
        for _ in range(2):
            rank, out, err = q.get(timeout=120)
            assert err is None, err
            res[rank] = out
    finally:
        for p in procs:
            p.join(timeout=30)
            if p.is_alive():
                p.kill()
    assert res[0]["a2a"] == ["0->0", "1->0"] and res[1]["a2a"] == ["0->1", "1->1"]
    assert res[0]["gathered"] == [0, 1] == res[1]["gathered"]
    assert res[0]["gather_dst1"] is None and res[1]["gather_dst1"] == [0, 1]
    assert res[1]["recv"] == ([0.0, 1.0, 2.0], "m", [1, 1], "torch.int64")
    assert res[0]["map"] == [10, 20, 30, 40, 50] == res[1]["map"]
    assert sorted(res[0]["did"] + res[1]["did"]) == [1, 2, 3, 4, 5] and res[0]["did"] and res[1]["did"]
    assert res[0]["bcast"] == ([1, 2, 3, 4], "hello") == res[1]["bcast"]
    assert res[0]["balanced"] == [0, 1, 2] and res[1]["balanced"] == [3, 4, 5]
    assert res[0]["restored"] == [0, 1, 2, 3, 4] and res[1]["restored"] == [5]
    assert res[0]["bmap"] == [100, 101, 102, 103, 104] and res[1]["bmap"] == [105]
    assert res[0]["concat"] == [0, 0, 1, 1] == res[1]["concat"]
    assert res[0]["concat_one"] == [0, 1, 2] == res[1]["concat_one"]
    assert res[0]["gather_obj"] == [[], []] and res[1]["gather_obj"] == [["from0"], ["from1"]]
    assert res[0]["a2a_tensors"] == [((1, 1), 0.0), ((2, 1), 10.0)] and res[1]["a2a_tensors"] == [((1, 2), 1.0), ((2, 2), 11.0)]
    assert res[1]["recv_obj"] == ([1, 2], [1.0, 1.0])
    assert res[1]["recv_packed"] == ((3, 1), [0, 1, 2], None)


def test_links_modules_placeholders_and_progress(tmp_path, capsys):
    import io
    import os
    import pickle

    from steptronoss_b200.utils import general as g

    (tmp_path / "data").mkdir()
    g.check_and_link(str(tmp_path / "data") + "/", str(tmp_path / "link"))
    g.check_and_link(str(tmp_path / "data"), str(tmp_path / "link"))            # same target again: fine
    assert os.readlink(tmp_path / "link") == str(tmp_path / "data")
    with pytest.raises(OSError):
        g.check_and_link(str(tmp_path / "other"), str(tmp_path / "link"))
    assert g.try_save({"a": 1}, str(tmp_path / "no" / "such" / "dir" / "x.pt")) is None       # logged, not raised
    g.try_save({"a": torch.ones(2)}, str(tmp_path / "x.pt"))
    assert torch.load(tmp_path / "x.pt")["a"].sum() == 2
    assert g.get_object_from_file("steptronoss_b200/utils/general.py", "safediv") is g.safediv

    calls = []

    @g.deprecated("use new_thing")
    def old_thing(x):
        calls.append(x)
        return x + 1

    assert old_thing(1) == 2 and old_thing(2) == 3 and calls == [1, 2]

    blob = pickle.dumps(g.safediv).replace(b"safediv", b"gone_fn")              # a dump that names something removed
    saved = (pickle.Unpickler, pickle._Unpickler.find_class)
    try:
        g.hack_pickle_load()
        g.hack_pickle_load()                                                    # patching twice changes nothing
        assert pickle._Unpickler(io.BytesIO(blob)).load().__name__ == "LoadFailure"
        assert "Cannot Load" in capsys.readouterr().out
    finally:
        pickle.Unpickler, pickle._Unpickler.find_class = saved                  # the patch is process-wide: undo it

    bars = g.GroupedProgressBar({"a": 2, "b": 1})
    bars.update("a")
    bars.update("b")
    assert bars.total_bar.n == 2 and bars.group_bars["a"].n == 1
    bars.close()


def test_gae_by_coefficient_matrix_matches_the_recursion():
    from steptronoss_b200.utils.rl_utils import compute_gae, compute_gae_opt, gae_coefficients

    torch.manual_seed(0)
    v, r = torch.randn(3, 9), torch.randn(3, 9)
    want = compute_gae(v, r, 0.9, 0.99)
    got = compute_gae_opt(v, r, 0.9, 0.99, gae_coeff=gae_coefficients(16, 0.9, 0.99))
    assert torch.allclose(got[0], want[0], atol=1e-5) and torch.allclose(got[1], want[1], atol=1e-5)
    same = compute_gae_opt(v, r, 0.9, 0.99)
    assert torch.equal(same[0], want[0])


def test_objects_as_byte_tensors_and_metric_axis_names():
    from steptronoss_b200.utils.dist_utils import object_to_tensor, tensor_to_object
    from steptronoss_b200.utils.metrics import Metric, RDims, ROps

    data, size = object_to_tensor({"a": [1, 2, torch.ones(2)]}, "cpu")
    assert data.dtype == torch.uint8 and int(size) == data.numel()
    padded = torch.cat([data, torch.zeros(7, dtype=torch.uint8)])            # as after a padded all-gather
    back = tensor_to_object(padded, size)
    assert back["a"][:2] == [1, 2] and back["a"][2].tolist() == [1.0, 1.0]
    m = Metric()._link(ROps.sum, RDims.time)
    m.add(1)
    m.add(2)
    assert float(m.reduce()) == 3.0 and RDims._get_group(RDims.world) is None
