"""Rule language of the HF weight loader: rename with captures, rank slices, concatenation, sharded writer."""
import json
import os

import pytest
import torch

from steptronoss_b200.utils.weight_loader import HFWeights, fill_target, key_pattern, parse_rules, write_safetensors


def _ckpt(tmp_path):
    torch.manual_seed(0)
    t = {}
    for i in range(2):
        for n, shape in (("q_proj", (8, 4)), ("k_proj", (4, 4)), ("v_proj", (4, 4)), ("o_proj", (4, 8))):
            t[f"transformer.model.layers.{i}.self_attn.{n}.weight"] = torch.randn(*shape)
    t["transformer.model.norm.weight"] = torch.randn(4)
    t["lm_head.weight"] = torch.randn(16, 4)
    write_safetensors(t, str(tmp_path / "src"), shard_max_size=200)   # forces several shards
    return t, HFWeights(str(tmp_path / "src"))


def test_patterns_and_targets():
    m = key_pattern("a.*.b.**.c?").match("a.1.b.xy.z.c9")
    assert m and m.groups() == ("1", "xy.z")
    assert fill_target(m, "n.*.m.*") == "n.1.m.xy.z"
    assert fill_target(m, "$2/$1") == "xy.z/1"
    assert key_pattern("a.b").match("axb") is None      # '.' is literal
    with pytest.raises(ValueError):
        fill_target(m, "*.*.*")


def test_sharded_round_trip(tmp_path):
    t, w = _ckpt(tmp_path)
    files = [f for f in os.listdir(tmp_path / "src") if f.endswith(".safetensors")]
    assert len(files) > 2 and set(w.keys()) == set(t)
    index = json.load(open(tmp_path / "src" / "model.safetensors.index.json"))
    assert index["metadata"]["total_size"] == sum(v.numel() * 4 for v in t.values())
    for k, v in t.items():
        assert torch.equal(w[k], v)


def test_export_rename_and_concatenate(tmp_path):
    t, w = _ckpt(tmp_path)
    out = w.export("""
        model.*: transformer.model.*
        *wqkv.weight CAT(0) *q_proj.weight *k_proj.weight *v_proj.weight
    """)
    assert "model.norm.weight" in out and "lm_head.weight" in out
    assert not any("q_proj" in k or "transformer." in k for k in out)
    for i in range(2):
        pre = f"transformer.model.layers.{i}.self_attn."
        want = torch.cat([t[pre + "q_proj.weight"], t[pre + "k_proj.weight"], t[pre + "v_proj.weight"]], 0)
        assert torch.equal(out[f"model.layers.{i}.self_attn.wqkv.weight"], want)
        assert torch.equal(out[f"model.layers.{i}.self_attn.o_proj.weight"], t[pre + "o_proj.weight"])
    w.write_safetensors_to(str(tmp_path / "dst"), tensors=out)
    again = HFWeights(str(tmp_path / "dst"))
    assert set(again.keys()) == set(out) and torch.equal(again["lm_head.weight"], t["lm_head.weight"])


def test_export_rank_slice_and_dict_rules(tmp_path):
    from steptronoss_b200.parallel.state import PM
    from steptronoss_b200.utils.weight_loader import Cat, Is

    t, w = _ckpt(tmp_path)
    PM.new_parallel("TP", [[0]])
    out = w.export({"head.weight": Is("lm_head.weight|TP@0"),
                    "*.kv": Cat("*.k_proj.weight", "*.v_proj.weight", dim=1, pop=False)})
    assert torch.equal(out["head.weight"], t["lm_head.weight"])
    k0 = "transformer.model.layers.0.self_attn"
    assert out[k0 + ".kv"].shape == (4, 8) and k0 + ".k_proj.weight" in out
    rules = parse_rules(["a.*: b.*|TP@1", "x: CAT(1) y z"])
    assert rules["a.*"].slice == ("TP", 1) and rules["x"].dim == 1 and rules["x"].components == ("y", "z")
