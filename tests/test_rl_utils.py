"""RL helpers: running moments, GAE against the textbook recursion, the sample dumper and the acknowledged queues."""
import os
import types

import pytest
import torch


def test_running_moments_match_the_whole_stream():
    from steptronoss_b200.utils.rl_utils import RunningMoments

    torch.manual_seed(0)
    xs = torch.randn(1000) * 3 + 2
    rm = RunningMoments()
    for part in xs.split(250):
        mean, std = rm.update(part)
        assert float(mean) == pytest.approx(float(part.mean()), abs=1e-5) and float(std) == pytest.approx(float(part.std()), rel=1e-4)
    assert float(rm.mean) == pytest.approx(float(xs.mean()), abs=1e-4)
    assert float(rm.std) == pytest.approx(float(xs.std()), rel=1e-3)


def test_gae_is_the_discounted_sum_of_td_errors():
    from steptronoss_b200.utils.rl_utils import compute_gae

    torch.manual_seed(1)
    v, r = torch.randn(7), torch.randn(7)
    gamma, lam = 0.9, 0.8
    adv, ret = compute_gae(v, r, lam, gamma)
    want = []
    for t in range(7):
        acc = 0.0
        for k in range(t, 7):
            nxt = float(v[k + 1]) if k + 1 < 7 else 0.0
            acc += (gamma * lam) ** (k - t) * (float(r[k]) + gamma * nxt - float(v[k]))
        want.append(acc)
    assert torch.allclose(adv, torch.tensor(want), atol=1e-5) and torch.allclose(ret, adv + v)
    cu = torch.tensor([0, 3, 3, 7], dtype=torch.int32)             # two segments and an empty one
    a2, r2 = compute_gae(v, r, lam, gamma, cu)
    a_first, _ = compute_gae(v[:3], r[:3], lam, gamma)
    a_second, ret_second = compute_gae(v[3:], r[3:], lam, gamma)
    assert torch.allclose(a2[:3], a_first) and torch.allclose(a2[3:], a_second) and torch.allclose(r2[3:], ret_second)
    batch_adv, _ = compute_gae(torch.stack([v, v * 2]), torch.stack([r, r]), lam, gamma)
    assert torch.allclose(batch_adv[0], adv)


def test_distributed_dict_list_merges_local_entries():
    from steptronoss_b200.utils.rl_utils import DistributedDictList

    d = DistributedDictList()
    with d.in_local():
        d["reward"] += [1.0, 2.0]
        d["len"] += [5]
    with d.in_local():
        d["reward"] += [3.0]
    assert d["reward"] == [1.0, 2.0, 3.0] and d["len"] == [5]


def test_sample_dumper_cuts_packed_tensors_by_generated_tokens():
    from steptronoss_b200.utils.rl_utils import RaggedPPOSampleDumper

    samples = [types.SimpleNamespace(meta={"id": i}, trajectory=[0] * n) for i, n in enumerate((4, 3))]
    packed = types.SimpleNamespace(
        samples=samples, cu_seqlens=torch.tensor([0, 4, 7]),
        is_gen_mask=torch.tensor([0, 0, 1, 1, 0, 1, 1]),            # 2 generated tokens each
        advantages=torch.tensor([1.0, 2.0, 3.0, 4.0]), values=None)
    out = RaggedPPOSampleDumper()([packed], ["trajectory", "advantages"])
    assert [o["meta"]["id"] for o in out] == [0, 1]
    assert out[0]["advantages"].tolist() == [1.0, 2.0] and out[1]["advantages"].tolist() == [3.0, 4.0]
    assert out[1]["trajectory"] == [0, 0, 0]


def test_acknowledged_queue_source_dumper_and_flow(tmp_path):
    from steptronoss_b200.utils.rl_utils import PersistentDumper, PersistentFlow, PersistentQueue, PersistentSource

    q = PersistentQueue()
    q.put("a", "b", "c")
    k1, first = q.get()
    k2, second = q.get()
    assert (first, second) == ("a", "b") and len(q) == 1 and not q.all_done()
    q.ack(k1)
    restored = PersistentQueue.from_state_dict(q.state_dict())       # "b" was taken but never acknowledged
    assert [restored.get()[1] for _ in range(2)] == ["b", "c"]
    q.ack(k2)
    q.ack(q.get()[0])
    assert q.empty() and q.all_done() and "PersistentQueue" in repr(q)

    class Count:
        def __init__(self):
            self.i = 0

        def __next__(self):
            self.i += 1
            return self.i

        def state_dict(self):
            return {"i": self.i}

        def load_state_dict(self, sd):
            self.i = sd["i"]

    src = PersistentSource(Count())
    ka, a = src.get()
    kb, b = src.get()
    src.ack(ka)
    state = src.state_dict()
    again = PersistentSource(Count())
    again.load_state_dict(state)
    assert [again.get()[1] for _ in range(2)] == [2, 3]              # the unacknowledged item first, then new ones
    with pytest.raises(RuntimeError):
        src.put(1)

    sink = PersistentDumper(str(tmp_path / "dump"), dump_interval=2)
    for i in range(5):
        sink.put({"i": i})
    files = sorted(os.listdir(tmp_path / "dump"))
    assert files == ["pdump_0.pt", "pdump_1.pt"] and sink.state_dict() == [{"i": 4}]
    assert [d["i"] for d in torch.load(tmp_path / "dump" / "pdump_1.pt", weights_only=False)] == [3, 2]
    assert PersistentDumper(str(tmp_path / "dump"), 2).dump_counter == 2     # a restart continues the numbering
    with pytest.raises(RuntimeError):
        sink.get()

    flow = PersistentFlow(meta={"version": 3}, todo=PersistentQueue(), done=PersistentQueue())
    flow["todo"].put(1, 2)
    with flow.lock:
        key, item = flow["todo"].get()
        flow["done"].put(item)
        flow["todo"].ack(key)
    snap = flow.state_dict()
    other = PersistentFlow(todo=PersistentQueue(), done=PersistentQueue())
    other.load_state_dict(snap)
    assert other.meta == {"version": 3} and other["todo"].state_dict() == [2] and other["done"].state_dict() == [1]
    sig = PersistentFlow.Signal("stop", reason="x")
    assert sig.name == "stop" and sig["reason"] == "x"
