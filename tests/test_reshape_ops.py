"""HF <-> native weight mapping: op algebra round trips and a full Qwen3 model round trip through safetensors."""
import torch

from steptronoss_b200.checkpointing import reshape_ops as R


def test_sequential_inverse_and_rename():
    op = R.VocabPad(10, 0) + R.ColumnParallel() + R.KeepThisTP() + R.Rename("dst.w: src.w")
    piece = {"src.w": torch.arange(16.0).view(8, 2)}
    out = op.forward(piece)
    assert list(out) == ["dst.w"] and out["dst.w"].shape == (10, 2)
    back = op.backward(out)
    assert torch.equal(back["src.w"], piece["src.w"])
    assert torch.equal(R.Inverse(op).backward(piece)["dst.w"], out["dst.w"])


def test_gqa_merge_and_ffn_merge_round_trip_with_fake_tp(monkeypatch):
    monkeypatch.setattr(R, "_size", lambda g: 2)
    monkeypatch.setattr(R, "_rank", lambda g: 1)
    hq, hkv, D, H = 4, 2, 8, 16
    piece = {"l.self_attn.q_proj.weight": torch.randn(hq * D, H), "l.self_attn.k_proj.weight": torch.randn(hkv * D, H),
             "l.self_attn.v_proj.weight": torch.randn(hkv * D, H)}
    op = R.GQAMergeQKV(hkv, D)
    merged = op.forward(piece)
    shards = merged["l.self_attn.qkv_proj.weight"]
    assert len(shards) == 2 and shards[0].shape == ((hq + 2 * hkv) * D // 2, H)
    # rank 1 shard = [q heads 2,3 | k head 1 | v head 1]
    assert torch.equal(shards[1][: 2 * D], piece["l.self_attn.q_proj.weight"][2 * D:])
    assert torch.equal(shards[1][2 * D: 3 * D], piece["l.self_attn.k_proj.weight"][D:])
    back = op.backward(merged)
    for k in piece:
        assert torch.equal(back[k], piece[k])
    ffn = {"l.mlp.gate_proj.weight": torch.randn(12, H), "l.mlp.up_proj.weight": torch.randn(12, H)}
    fop = R.FFNMergeGateUp()
    m2 = fop.forward(ffn)
    assert torch.equal(m2["l.mlp.gate_up_proj.weight"][0], torch.cat([ffn["l.mlp.gate_proj.weight"][:6], ffn["l.mlp.up_proj.weight"][:6]]))
    b2 = fop.backward(m2)
    assert all(torch.equal(b2[k], ffn[k]) for k in ffn)


def test_unbind_moe_round_trip():
    piece = {f"m.experts.{i}.down_proj.weight": torch.full((2, 3), float(i)) for i in range(4)}
    op = R.UnbindMoE("experts.")
    st = op.forward(piece)
    assert st["m.experts.down_proj.weight"].shape == (4, 2, 3)
    back = op.backward(st)
    assert all(torch.equal(back[k], piece[k]) for k in piece)


def test_qwen_model_hf_round_trip(tmp_path):
    from playground.pretrain.qwen3.qwen3_8b import Qwen3_8BConfig
    from steptronoss_b200.checkpointing.hf_checkpoint import HFWeights, dump_safetensors

    cfg = Qwen3_8BConfig()
    cfg.num_layers, cfg.hidden_size, cfg.params_dtype = 2, 64, torch.float32
    cfg.parallel_cfg.tensor_model_parallel_size = 1
    cfg.tp_cfg.sequence_parallel = False
    a = cfg.attn_cfg
    a.num_attention_heads, a.num_attention_groups, a.head_dim, a.hidden_size = 4, 2, 16, 64
    cfg.ffn_cfg.hidden_size, cfg.ffn_cfg.ffn_hidden_size = 64, 96
    cfg.tok_embed_cfg.vocab_size = cfg.out_embed_cfg.vocab_size = 128
    cfg.tok_embed_cfg.hidden_size = cfg.out_embed_cfg.hidden_size = 64
    m = cfg.build_model()
    m.init_weights(1)
    hf = m.hf_state_dict()
    assert "model.layers.1.self_attn.k_proj.weight" in hf and "model.layers.0.mlp.up_proj.weight" in hf
    assert hf["model.layers.0.self_attn.q_proj.weight"].shape == (64, 64) and hf["lm_head.weight"].shape == (128, 64)
    dump_safetensors([m], str(tmp_path))
    m2 = cfg.build_model()
    m2.init_weights(2)
    m2.load_hf_state_dict(HFWeights(str(tmp_path)))
    for (n, p), (_, q) in zip(m.named_parameters(), m2.named_parameters()):
        assert torch.equal(p, q), n


def test_qkv_bias_trains_and_round_trips_through_the_hf_layout():
    """``use_qkv_bias`` (Qwen2-style): the fused projection gets a bias that starts at zero, receives gradients, and
    maps to ``q_proj.bias / k_proj.bias / v_proj.bias`` and back."""
    import torch

    from steptronoss_b200.models.qwen_dense import QwenModel
    from steptronoss_b200.parallel.state import PM
    from tests.tiny_exp import make_tiny_exp

    PM.initialize()
    exp = make_tiny_exp(gbs=1, seq=32, iters=1, layers=1, hidden=32, heads=4, kv_heads=2, head_dim=8, ffn=64, vocab=64)
    cfg = exp.model_cfg
    cfg.attn_cfg.use_qkv_bias = True
    PM.set_mesh(cfg.parallel_cfg)
    model = QwenModel(cfg=cfg, layer_map=cfg.build_layer_map())
    model.init_weights(0, 0.02)
    bias = model.layers["0"].attention.wqkv.bias
    assert bias.shape == (4 * 8 + 2 * 2 * 8,) and float(bias.abs().sum()) == 0.0
    ids = torch.randint(0, 64, (1, 32))
    out = model(input_ids=ids, labels=ids, cu_seqlens=torch.tensor([0, 32], dtype=torch.int32), max_seq_len=32,
                position_id=torch.arange(32, dtype=torch.int32))
    (out["loss"] if isinstance(out, dict) else out.float().mean()).backward()
    assert bias.grad is not None and float(bias.grad.abs().sum()) > 0
    with torch.no_grad():
        bias.copy_(torch.arange(64.0))
    hf = model.hf_state_dict()
    q, k, v = (hf[f"model.layers.0.self_attn.{n}_proj.bias"] for n in "qkv")
    assert q.tolist() == list(range(32)) and k.tolist() == list(range(32, 48)) and v.tolist() == list(range(48, 64))
    other = QwenModel(cfg=cfg, layer_map=cfg.build_layer_map())
    other.init_weights(1, 0.02)
    other.load_hf_state_dict(hf)
    assert torch.equal(other.layers["0"].attention.wqkv.bias, bias)
