"""RoPE tables and rotation (fp32 caches, partial rotary, position ids, YaRN), metric reductions, indexed-bin /
compiled / chat-JSON datasets with the chat template, multimodal input helpers."""
import json
import os

import numpy as np
import pytest
import torch


# ------------------------------------------------------------------------------------------------ RoPE
def test_rope_tables_stay_fp32_and_grow():
    from steptronoss_b200.models.common.rope import RotaryEmbedding

    r = RotaryEmbedding(rot_dim=64, theta=1e4, max_position=128)
    cos, sin = r.tables(torch.device("cpu"))
    assert cos.dtype == torch.float32 and cos.shape[1] == 32 and cos.shape[0] >= 128
    r = r.to(torch.bfloat16)                              # casting the model must not touch the caches
    cos2, _ = r.tables(torch.device("cpu"), need=100000)
    assert cos2.dtype == torch.float32 and cos2.shape[0] >= 100000
    pos = torch.tensor([0, 1, 77])
    want = torch.cos(pos[:, None].double() * (1.0 / 1e4 ** (torch.arange(0, 64, 2).double() / 64))[None]).float()
    assert torch.allclose(cos2[pos], want, atol=1e-6)


def test_rotation_is_half_split_relative_and_partial():
    from steptronoss_b200.ops import rope_tables
    from steptronoss_b200.ops.fused import qknorm_rope_reference

    D, hq, hkv, T = 16, 2, 1, 6
    torch.manual_seed(0)
    qkv = torch.randn(T, (hq + 2 * hkv) * D)
    cos, sin = rope_tables(64, D, 1e4, torch.device("cpu"))
    pos = torch.arange(T)
    q, k, v = qknorm_rope_reference(qkv, None, None, cos, sin, pos, hq, hkv, D, use_norm=False)
    x = qkv[:, :D]                                         # head 0 of q before rotation
    x1, x2 = x[:, : D // 2], x[:, D // 2:]
    c, s = cos[pos], sin[pos]
    assert torch.allclose(q[:, 0], torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], -1), atol=1e-5)   # half-split pairs
    assert torch.allclose(v.reshape(T, -1), qkv[:, (hq + hkv) * D:])                                  # v untouched
    # scores depend on the position difference only
    q5, k5, _ = qknorm_rope_reference(qkv, None, None, cos, sin, pos + 5, hq, hkv, D, use_norm=False)
    assert torch.allclose(q[:, 0] @ k[:, 0].T, q5[:, 0] @ k5[:, 0].T, atol=1e-4)
    # packed documents: position ids restart, so token 3 of the second document rotates like position 0
    pid = torch.tensor([0, 1, 2, 0, 1, 2])
    qp, _, _ = qknorm_rope_reference(qkv, None, None, cos, sin, pid, hq, hkv, D, use_norm=False)
    assert torch.allclose(qp[3, 0], qkv[3, :D], atol=1e-6)
    # partial rotary: the tail of every head passes through
    cos8, sin8 = rope_tables(64, 8, 1e4, torch.device("cpu"))
    qr, kr, _ = qknorm_rope_reference(qkv, None, None, cos8, sin8, pos, hq, hkv, D, rot_dim=8, use_norm=False)
    assert torch.allclose(qr[:, 1, 8:], qkv[:, D + 8: 2 * D]) and not torch.allclose(qr[1:, 1, :8], qkv[1:, D: D + 8])


def test_yarn_blends_interpolated_and_extrapolated_frequencies():
    from steptronoss_b200.models.common.rope import yarn_inv_freq

    rot, theta = 64, 1e4
    base = 1.0 / (theta ** (torch.arange(0, rot, 2, dtype=torch.float64) / rot))
    assert torch.equal(yarn_inv_freq(base, rot, theta, 1.0, 4096), base)
    y = yarn_inv_freq(base, rot, theta, 4.0, 4096)
    assert torch.allclose(y[0], base[0]) and torch.allclose(y[-1], base[-1] / 4.0)      # fast dims kept, slow dims / 4
    assert bool(((y <= base + 1e-18) & (y >= base / 4.0 - 1e-18)).all())
    ratio = y / base
    assert bool((ratio[1:] <= ratio[:-1] + 1e-12).all())                                # monotone ramp


# ------------------------------------------------------------------------------------------------ metrics
def test_metric_chains_percentages_groups_and_holder():
    from steptronoss_b200.utils.metrics import (AvgMetric, GroupMetric, HistogramMetric, Metric, MetricHolder,
                                                PercentageMetric, TextMetric)

    m = Metric().sum("time")
    for v in (1.0, 2.0, torch.tensor(3.0)):
        m.add(v)
    assert float(m.reduce()) == 6.0
    assert float(Metric().reduce() or 0.0) == 0.0
    mx = Metric().max("time")
    mx.add(torch.tensor([1.0, 5.0]), iop=torch.max)          # an input transform
    mx.add(2.0)
    mx.add(4.0, iop="max")                                   # merged into the last value
    assert float(mx.reduce()) == 5.0 and len(mx.values) == 2
    last = Metric().last("time")
    last.add(1.0)
    last.add(9.0)
    assert float(last.reduce()) == 9.0
    p = PercentageMetric().mean("time")
    p.add(1, 4)
    p.add(3, 4)
    assert float(p.reduce()) == pytest.approx(0.5)           # (1 + 3) / (4 + 4), not the mean of the ratios
    cats = PercentageMetric()
    cats.add(3, subname="stop")
    cats.add(1, subname="length")
    assert {k: float(v) for k, v in cats.reduce().items()} == {"length": 0.25, "stop": 0.75}
    g = Metric(is_group=True).mean("time")
    assert isinstance(g, GroupMetric)
    g.add(1.0, subname="layer0")
    g.add(3.0, subname="layer0")
    g.add(5.0, subname="layer1")
    assert {k: float(v) for k, v in g.reduce().items()} == {"layer0": 2.0, "layer1": 5.0}
    h = HistogramMetric()
    h.add(torch.arange(3.0))
    h.add(torch.tensor([7.0]))
    assert h.reduce().tolist() == [0.0, 1.0, 2.0, 7.0]
    t = TextMetric(2)
    for s in ("a", "b", "c"):
        t.add(s)
    assert t.reduce() == ["a", "b"]
    holder = MetricHolder()
    holder.register("loss", Metric().mean("time"))
    holder.register("per_layer", g)
    holder.loss.add(2.0)
    holder.not_registered.add(1.0)                            # unknown names swallow values
    with holder.disable():
        holder.loss.add(100.0)
    with holder.fork():
        holder.loss.add(50.0)
        assert float(holder.reduce_all()["loss"]) == 50.0
    out = holder.reduce_all()
    assert float(out["loss"]) == 2.0 and set(out) == {"loss", "per_layer/layer0", "per_layer/layer1"}
    assert holder.reduce_all().get("loss") is None or "loss" not in holder.reduce_all()    # reset after reduce


# ------------------------------------------------------------------------------------------------ datasets
class _Tok:
    chat_template = None

    def encode(self, text, add_special_tokens=False):
        return [ord(c) % 251 for c in text]


def test_indexed_bin_compiled_and_chat_datasets(tmp_path):
    from steptronoss_b200.data.chat_template import HuggingFaceTemplate
    from steptronoss_b200.data.datasets import CompiledDataset, StepChatJsonDataset, compile_dataset
    from steptronoss_b200.data.indexed_bin import IndexedBinReader, IndexedBinWriter

    with IndexedBinWriter(str(tmp_path / "bin"), cfg={"note": "x"}) as w:
        ids = [w.append({"i": i, "blob": np.arange(i)}) for i in range(5)]
    assert ids == list(range(5)) and os.path.exists(tmp_path / "bin" / ".success")
    r = IndexedBinReader(str(tmp_path / "bin"))
    assert len(r) == 5 and r[3]["i"] == 3 and r[4]["blob"].tolist() == [0, 1, 2, 3]
    with pytest.raises(IndexError):
        r[5]

    convs = [{"conversations": [{"role": "user", "content": f"q{i}"},
                                {"role": "assistant", "content": f"old{i}", "loss_mask": 1},
                                {"role": "user", "content": "again"},
                                {"role": "assistant", "content": [{"type": "text", "value": f"new{i}"}], "loss_mask": 1}]}
             for i in range(7)]
    convs[2]["conversations"][-1]["loss_mask"] = 0
    (tmp_path / "chat.json").write_text(json.dumps(convs))
    ds = StepChatJsonDataset(str(tmp_path / "chat.json"), template=HuggingFaceTemplate(_Tok()))
    assert len(ds) == 7
    s = ds[0]
    assert s["tokens"].dtype == np.int32 and s["loss_mask"].dtype == np.float16 and len(s["tokens"]) == len(s["loss_mask"])
    text = "".join(f"<|im_start|>{c['role']}\n{c['content'] if isinstance(c['content'], str) else c['content'][0]['value']}<|im_end|>\n"
                   for c in convs[0]["conversations"])
    assert s["tokens"].tolist() == _Tok().encode(text)
    trained = "".join(chr(t) for t, m in zip(s["tokens"].tolist(), s["loss_mask"].tolist()) if m)   # ascii survives % 251
    assert "new0" in trained and "old0" not in trained and "again" not in trained   # only turns after the last user turn
    assert float(ds[2]["loss_mask"].sum()) == 0.0                                    # loss_mask 0 switches a turn off
    manifest = compile_dataset(ds, str(tmp_path / "compiled"), n_shards=3)
    assert manifest["length"] == 7 and [x["size"] for x in manifest["shards"]] == [3, 2, 2]
    cd = CompiledDataset(str(tmp_path / "compiled"))
    assert len(cd) == 7 and cd.sample_length(5) == len(ds[5]["tokens"])
    for i in range(7):
        assert cd[i]["tokens"].tolist() == ds[i]["tokens"].tolist()
    with pytest.raises(FileNotFoundError):
        CompiledDataset(str(tmp_path))


def test_multimodal_inputs():
    from steptronoss_b200.data.multimodal import (IMAGE_ITEM_TYPE, PATCH_ITEM_TYPE, build_image_for_insert,
                                                 compute_rope_args)

    items = [(torch.zeros(3, 28, 28), IMAGE_ITEM_TYPE), (torch.ones(3, 28, 28), PATCH_ITEM_TYPE),
             (torch.ones(3, 28, 28), PATCH_ITEM_TYPE), (torch.zeros(3, 28, 28), IMAGE_ITEM_TYPE)]
    out = build_image_for_insert(items, patch_start_id=11, image_start_id=22, limit_patches=1, dtype=torch.float32,
                                 to_cuda=False, rope_args_fn=lambda ts: compute_rope_args(ts, 14, to_cuda=False))
    assert [o.insert_start_token for o in out] == [11, 22] and out[0].images.shape == (1, 3, 28, 28)
    assert out[1].images.shape == (2, 3, 28, 28) and out[1].rope_cu_seqlens.tolist() == [0, 4, 8] and out[1].rope_max_seq_len == 4
    with pytest.raises(ValueError):
        build_image_for_insert([(torch.zeros(1), 9)], patch_start_id=1, image_start_id=2)
    with pytest.raises(ValueError):
        compute_rope_args([], 14, to_cuda=False)


def test_dialog_types_and_validation():
    from steptronoss_b200.data.types import MessageContentType, Role, validate_dialog

    assert Role.ASSISTANT == "assistant" and MessageContentType.TEXT.value == "text"
    good = {"conversations": [{"role": "user", "content": "hi"},
                              {"role": "assistant", "content": [{"type": "text", "value": "yo", "loss_mask": 1}], "loss_mask": 1}]}
    assert validate_dialog(good) == []
    bad = {"conversations": [{"role": "robot", "content": 3}, {"role": "user", "content": [{"type": "video", "value": "x"}], "loss_mask": 2}]}
    probs = validate_dialog(bad)
    assert len(probs) == 5 and any("robot" in p for p in probs) and any("no assistant turn" in p for p in probs)
    assert validate_dialog({}) == ["'conversations' must be a non-empty list"]


def test_outlier_metric_dumps_the_data_of_values_above_the_recent_mean(tmp_path):
    import torch

    from steptronoss_b200.utils.metrics import DummyMetric, GlobalMetrics, WithDataDumpOutlierMetric, dummy_metric

    m = WithDataDumpOutlierMetric(max_window_size=3, outlier_data_dump_dir=str(tmp_path))
    for step in range(3):                                   # the window fills: nothing is an outlier yet
        m.add({"real_value": 1.0 + 0.01 * step, "data": {"step": step}})
        assert float(m.reduce()) == 0.0
        m.reset()
    m.add({"real_value": 0.9, "data": {"step": 3}})
    m.add({"real_value": 5.0, "data": {"step": 4, "ids": torch.arange(3)}})
    assert float(m.reduce()) == 1.0 and len(m.dumped) == 1
    saved = torch.load(m.dumped[0], weights_only=False)
    assert saved["real_value"] == 5.0 and saved["data"]["step"] == 4 and saved["data"]["ids"].tolist() == [0, 1, 2]
    m.reset()
    assert float(m.reduce()) == 0.0
    import pytest

    with pytest.raises(ValueError):
        m.add({"value": 1})
    assert isinstance(dummy_metric, DummyMetric) and GlobalMetrics.some_metric_nobody_registered is dummy_metric
    dummy_metric.add(1, subname="x")


def _pooled_worker(rank, world):
    from steptronoss_b200.exp.base_exp import ParallelConfig
    from steptronoss_b200.parallel.state import PM
    from steptronoss_b200.utils.metrics import AvgMetric, Metric

    PM.set_mesh(ParallelConfig())                                        # two data-parallel ranks
    pooled, plain = AvgMetric().mean("world"), Metric().mean("time").mean("world")
    spread, top = AvgMetric().std("world"), AvgMetric().max("dp")
    for v in ([1.0] if rank == 0 else [3.0, 3.0, 3.0]):                  # one sample here, three there
        for m in (pooled, plain, spread, top):
            m.add(v)
    return float(pooled.reduce()), float(plain.reduce()), float(spread.reduce()), float(top.reduce())


def test_avg_metric_pools_samples_over_ranks():
    from steptronoss_b200.utils.metrics import AvgMetric
    from tests.dist_helpers import call_on_ranks

    got = call_on_ranks(_pooled_worker, 2)
    for rank in (0, 1):
        pooled, plain, spread, top = got[rank]
        assert pooled == 2.5 and plain == 2.0                               # per-sample mean against mean of means
        assert spread == pytest.approx(1.0) and top == 3.0
    one = AvgMetric().std("world")
    one.add(2)
    assert float(one.reduce()) == 0.0 and AvgMetric().mean("world").reduce() is None
    with pytest.raises(ValueError):
        m = AvgMetric().sum("world")
        m.add(1.0)
        m.reduce()
