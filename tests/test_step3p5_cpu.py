"""Step-3.5 decoder on CPU: sliding-window and full-attention layers, routed experts with a shared expert,
head-wise attention gate; one training step and the HF <-> native weight mapping round trip."""
import pytest
import torch

from steptronoss_b200.data.synthetic import SyntheticDataConfig
from steptronoss_b200.exp.base_exp import GradientManagerConfig, ProfilerConfig
from steptronoss_b200.exp.lr_schedulers import ConstantSchedulerConfig
from steptronoss_b200.exp.ntp import NTPTrainerConfig, PretrainExp, PretrainMetricConfig
from steptronoss_b200.models.step3p5 import Step3p5Block, Step3p5ModelConfig


class _Exp(PretrainExp):
    trainer_cfg = NTPTrainerConfig
    model_cfg = Step3p5ModelConfig
    optimizer_cfg = GradientManagerConfig
    scheduler_cfg = ConstantSchedulerConfig
    data_cfg = SyntheticDataConfig
    metric_cfg = PretrainMetricConfig
    profiler_cfg = ProfilerConfig


def _make(layers=3, hidden=64, vocab=256):
    e = _Exp()
    m = e.model_cfg
    m.num_layers, m.hidden_size, m.params_dtype = layers, hidden, torch.float32
    m.variable_seq_lengths = True
    m.swa_layer_list = [True, False, True][:layers]
    for a, heads, window in ((m.attn_cfg, 4, None), (m.swa_cfg, 8, 16)):
        a.num_attention_heads, a.num_attention_groups, a.head_dim, a.hidden_size = heads, 2, 16, hidden
        a.rope_theta, a.use_qk_norm, a.use_headwise_attn_gate = 1e4, False, True
        if window:
            a.use_sliding_window, a.sliding_window_size = True, window
    f = m.ffn_cfg
    f.hidden_size, f.ffn_hidden_size = hidden, 96
    mc = m.moe_cfg
    mc.hidden_size, mc.moe_num_experts, mc.moe_top_k, mc.moe_hidden_size = hidden, 4, 2, 32
    mc.moe_layer_list = [1, 2]
    mc.share_expert_dim = 48
    mc.enable_sigmoid_router = True
    mc.enable_auxiliary_loss_free_load_balance = True
    mc.router_bias_update_rate = 1e-3
    m.tok_embed_cfg.vocab_size = m.out_embed_cfg.vocab_size = vocab
    m.tok_embed_cfg.hidden_size = m.out_embed_cfg.hidden_size = hidden
    m.parallel_cfg.expert_tensor_parallel_size = 1
    t = e.trainer_cfg
    t.global_batch_size, t.global_seq_length, t.train_iters, t.writer_backend = 2, 64, 4, []
    e.scheduler_cfg.lr, e.scheduler_cfg.weight_decay, e.scheduler_cfg.warmup_schedule = 1e-3, 0.0, 0
    e.data_cfg.min_doc_len, e.data_cfg.max_doc_len, e.data_cfg.pin_memory = 8, 32, False
    return e


def test_step3p5_layers_follow_the_swa_list_and_train():
    exp = _make()
    exp.seed = 0
    tr = exp.trainer_cfg.get_trainer_cls()(exp=exp)
    tr.before_train()
    model = tr.models[0]
    model = getattr(model, "module", model)
    blocks = [model.layers[str(i)] for i in model.layer_ids]
    assert all(isinstance(b, Step3p5Block) for b in blocks)
    assert [b.attention.window for b in blocks] == [17, 0, 17]       # 16 keys to the left and the query itself
    assert [b.attention.num_heads for b in blocks] == [8, 4, 8]
    assert not hasattr(blocks[0].feed_forward, "moe") and hasattr(blocks[1].feed_forward, "moe")
    assert blocks[1].feed_forward.enable_share_expert
    from steptronoss_b200.utils.metrics import GlobalMetrics, ModelLayerMetric

    GlobalMetrics.register("shared_routed_avgnorm", ModelLayerMetric().mean("time"))    # opt-in diagnostic
    losses = []
    for _ in range(4):
        tr.train_step()
        tr.iteration += 1
        tr.training_log()
        losses.append(tr.history[-1]["lm_loss"])
    assert all(l == l for l in losses) and losses[-1] < losses[0]
    norms = {k: float(v) for k, v in tr.last_metrics.items() if k.startswith("shared_routed_avgnorm/")}
    assert set(norms) == {f"shared_routed_avgnorm/layer{i}.{b}" for i in (0, 1) for b in ("routed", "shared")}
    assert all(v > 0 for v in norms.values())


def test_step3p5_hf_mapping_round_trip():
    exp = _make()
    exp.seed = 1
    tr = exp.trainer_cfg.get_trainer_cls()(exp=exp)
    tr.before_train()
    model = tr.models[0]
    model = getattr(model, "module", model)
    native = {k: v.detach().clone() for k, v in model.state_dict().items() if v is not None}
    hf = model.reshaper.backward({k: v for k, v in native.items()})
    assert "model.layers.0.self_attn.q_proj.weight" in hf and "model.layers.0.self_attn.g_proj.weight" in hf
    assert "model.layers.1.moe.gate_proj.weight" in hf and hf["model.layers.1.moe.gate_proj.weight"].shape == (4, 32, 64)
    assert "model.layers.1.share_expert.down_proj.weight" in hf and "model.layers.1.moe.router_bias" in hf
    back = model.reshaper.forward(hf)
    for k, v in native.items():
        if k in back:
            assert torch.equal(back[k], v), k
    assert set(back) >= {k for k in native if "rope" not in k and "tokens_per_expert" not in k}


def test_selection_bias_stays_fp32_through_casts_and_loads():
    exp = _make()
    exp.seed = 0
    tr = exp.trainer_cfg.get_trainer_cls()(exp=exp)
    tr.before_train()
    model = getattr(tr.models[0], "module", tr.models[0])
    moe = model.layers["1"].feed_forward.moe
    assert moe.router_balance_bias.dtype == torch.float32
    model.to(torch.bfloat16)
    assert moe.gate.weight.dtype == torch.bfloat16 and moe.router_balance_bias.dtype == torch.float32
    sd = {k: v.clone() for k, v in moe.state_dict().items()}
    sd["router_balance_bias"] = torch.full_like(sd["router_balance_bias"], 1.0 + 1e-3).to(torch.bfloat16)
    moe.load_state_dict(sd)
    assert moe.router_balance_bias.dtype == torch.float32
    assert model.pp_size == 1 and callable(model.abstract_forward)
    model.init_model_weight(seed=3)
    assert all(getattr(p, "has_initialized", False) for p in model.parameters())


def test_load_model_checkpoint_and_init_callback():
    import torch.nn as nn

    from steptronoss_b200.models.module import init_weight_callback, load_model_checkpoint

    exp = _make()
    exp.seed = 0
    tr = exp.trainer_cfg.get_trainer_cls()(exp=exp)
    tr.before_train()
    model = getattr(tr.models[0], "module", tr.models[0])
    saved = {k: v.detach().clone() for k, v in model.state_dict().items()}
    with torch.no_grad():
        for p in model.parameters():
            p.add_(1.0)
            p.has_initialized = False
    partial = {k: v for k, v in saved.items() if "tok_embeddings" not in k}
    load_model_checkpoint(tr.models, {"model": [partial]}, strict_load_model=False)
    named = dict(model.named_parameters())
    emb = next(k for k in named if "tok_embeddings" in k)
    other = next(k for k in named if "tok_embeddings" not in k)
    assert torch.equal(named[other], saved[other]) and named[other].has_initialized
    assert not torch.equal(named[emb], saved[emb]) and not named[emb].has_initialized       # was not in the checkpoint
    with pytest.raises(RuntimeError):
        load_model_checkpoint(tr.models, {"model": [partial]}, strict_load_model=True)
    with pytest.raises(AssertionError):
        load_model_checkpoint(tr.models, {})

    order = []

    class Leaf(nn.Module):
        def init_model_weight(self):
            order.append("leaf")

    @init_weight_callback
    class Net(nn.Module):
        def __init__(self):
            super().__init__()
            self.a = Leaf()

        def init_model_weight(self):
            order.append("net")

    class Bigger(Net):                                    # the callback belongs to Net's own instances
        pass

    Net()
    assert order == ["leaf", "net"]
    Bigger()
    assert order == ["leaf", "net"]
