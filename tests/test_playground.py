"""Every experiment file of the playground builds and passes its sanity check; the RLVR rollout item scores
completions; the standard evaluation set runs end to end with canned generations and resumes from its cache."""
import importlib
import json

import pytest

EXPERIMENTS = [
    ("playground.pretrain.qwen3.qwen3_8b", "Exp"), ("playground.pretrain.qwen3.qwen3_30a3b", "Exp"),
    ("playground.pretrain.debug", "Exp"),
    ("playground.sft.qwen3.qwen3_1p7b_sft", "Exp"), ("playground.sft.qwen3.qwen3_30a3b_sft", "Exp"),
    ("playground.sft.step3.step3_toy_sft", "Exp"), ("playground.sft.step3.step3_toy_sft_muon", "Exp"),
    ("playground.sft.step3.step3_toy_sft_muon_2node", "Exp"), ("playground.sft.step3.step3p5_flash_sft_muon", "Exp"),
    ("playground.rlvr.qwen3_1p5b_rlvr_math", "Exp"), ("playground.rlvr.qwen3_1p5b_rlvr_math_fully_async", "Exp"),
    ("playground.eval.qwen3.qwen3_eval_simple_benchmarks", "Exp"),
    ("playground.eval.qwen3.qwen3_eval_simple_benchmarks", "Exp1p7B"),
    ("playground.eval.step3p5.step3p5_eval_simple_benchmarks", "Exp"),
    ("playground.eval.step3v.step3v_eval_simple_benchmarks", "Exp"),
    ("playground.sft.step3v.step3v_10b_sft_tp8_caption_smoke", "Exp"),
]


@pytest.mark.parametrize("module,name", EXPERIMENTS, ids=[f"{m.split('.', 1)[1]}:{n}" for m, n in EXPERIMENTS])
def test_experiment_builds_and_is_sane(module, name):
    exp = getattr(importlib.import_module(module), name)()
    exp.sanity_check()
    d = exp.to_dict()
    assert isinstance(d, dict) and d
    json.dumps(exp.to_dict(rep=True), default=str)          # what the checkpoint and cfshow print


def test_model_configs_have_the_published_shapes():
    from playground.pretrain.qwen3.qwen3_1p7b import Qwen3_1p7BConfig
    from playground.pretrain.step3p5.step3p5_flash import Step3p5FlashModelConfig
    from playground.pretrain.step3p5.step3p5_toy import Step3p5ToyModelConfig

    q = Qwen3_1p7BConfig()
    assert (q.num_layers, q.hidden_size, q.attn_cfg.num_attention_heads, q.ffn_cfg.ffn_hidden_size, q.tie_embedding) == \
        (28, 2048, 16, 6144, True)
    f = Step3p5FlashModelConfig()
    assert len(f.swa_layer_list) == f.num_layers == 45 and sum(f.swa_layer_list) == 33
    assert f.swa_cfg.sliding_window_size == 512 and f.swa_cfg.num_attention_heads == 96 and f.attn_cfg.qk_rope_head_dim == 64
    assert f.moe_cfg.moe_layer_list[0] == 3 and f.moe_cfg.get_experts_swiglu_limit(44) == 7.0
    assert f.moe_cfg.get_experts_swiglu_limit(10) is None and f.moe_cfg.get_shared_expert_swiglu_limit(44) == 16.0
    t = Step3p5ToyModelConfig()
    t.sanity_check()
    assert t.moe_cfg.moe_num_experts == 128 and t.attn_cfg.hidden_size == 2048 and t.moe_cfg.get_experts_swiglu_limit(44) is None


def test_simple_trainable_scores_completions():
    from playground.rlvr.simple_trainable import SimpleTrainable
    from steptronoss_b200.exp.rl import StopType

    it = SimpleTrainable("q", "3", lambda: "http://x", lambda: "m", {"temperature": 0.5}, max_tokens=16)
    assert it.request()["temperature"] == 0.5 and it.request()["max_tokens"] == 16 and it.request()["model"] == "m"
    assert it.extract_boxed("so \\boxed{1} then \\boxed{ 3 }") == "3" and it.extract_boxed("none") == ""
    good = it.score({"prompt_token_ids": [1, 2], "token_ids": [3, 4, 5], "text": "it is \\boxed{3}", "finish_reason": "stop"})
    assert good.raw_reward == 1.0 and good.trajectory == [1, 2, 3, 4, 5] and good.is_gen_mask == [0, 0, 1, 1, 1]
    cut = it.score({"prompt_token_ids": [1], "token_ids": [3], "text": "\\boxed{3}", "finish_reason": "length"})
    assert cut.raw_reward == 0.0 and cut.stop_type == StopType.MAX_LEN
    wrong = it.score({"prompt_token_ids": [1], "token_ids": [3], "text": "\\boxed{4}", "finish_reason": "stop",
                      "logprobs": {"token_logprobs": [-0.5]}})
    assert wrong.raw_reward == 0.0 and wrong.logprobs == [-0.5]
    assert it.fingerprint() == SimpleTrainable("q", "3", None, None, {"temperature": 0.5}, 16).fingerprint()
    assert it.fingerprint() != SimpleTrainable("q2", "3", None, None, {"temperature": 0.5}, 16).fingerprint()


class _Tok:
    def apply_chat_template(self, msgs, tokenize=True, add_generation_prompt=True, **kw):
        return list(range(sum(len(m["content"].split()) for m in msgs)))

    def encode(self, text, add_special_tokens=False):
        return text.split()


def test_simple_eval_set_runs_and_resumes_from_its_cache(tmp_path, monkeypatch):
    from playground.eval.eval_sets import simple_eval as se
    from steptronoss_b200.exp import gen_eval
    from steptronoss_b200.generation.async_generation import SingleGenerationController
    from steptronoss_b200.generation.base_benchmark import Generated

    data = tmp_path / "data"
    (data / "AIME2025").mkdir(parents=True)
    rows = [{"dataset": "AIME2025", "messages": [{"role": "user", "content": f"what is {i} + {i}"}],
             "source_item": {"item_id": str(i), "answer": str(2 * i)}} for i in range(3)]
    (data / "AIME2025" / "test.jsonl").write_text("\n".join(json.dumps(r) for r in rows))
    (data / "IFBENCH").mkdir()
    (data / "IFBENCH" / "IFBench_test.jsonl").write_text(json.dumps(
        {"key": 7, "prompt": "no spaces please", "instruction_id_list": ["format:no_whitespace"], "kwargs": [{}]}))
    calls = []

    async def fake_generate(self):
        calls.append(self.case.benchmark.item_id)
        text = self.case.prompt.messages[-1]["content"]
        if self.case.benchmark.benchmark_name == "IFBENCH":
            return Generated(self.case, {"finish_reason": "stop"}, "nospaces")
        n = int(text.split()[2])
        if n == 2 and len([c for c in calls if c == "2"]) == 1:
            return Generated(self.case, error="TimeoutError: first try")
        return Generated(self.case, {"finish_reason": "stop"}, f"so \\boxed{{{2 * n if n != 1 else 99}}}")

    monkeypatch.setattr(gen_eval.ChatCaseGenable, "generate", fake_generate)
    monkeypatch.setattr(gen_eval.ChatCaseGenable, "payload", lambda self: ("/v1/chat/completions", {}))

    from steptronoss_b200.exp.base_exp import TokenizerConfig

    class Tok(TokenizerConfig):
        def build_tokenizer(self):
            return _Tok()

    class Cfg(se.SimpleBenchmarksEvalConfig):
        tokenizer_cfg = Tok

        def build_controller(self):
            return SingleGenerationController()

    cfg = Cfg()
    cfg.datasets_dir, cfg.save_dir = str(data), str(tmp_path / "out")
    cfg.sample_per_prompt = {"AIME2025": 1, "IFBENCH": 1}
    cfg.max_model_len, cfg.max_decode_steps = 100, 1000
    import steptronoss_b200.generation.base_generatable as bg
    monkeypatch.setattr(bg.EndpointGetter, "__call__", lambda self: "http://unused")
    monkeypatch.setattr(bg.ModelNameGetter, "__call__", lambda self: "m")
    s1 = cfg.eval()
    assert set(s1) == {"AIME2025", "IFBENCH"} and len(calls) == 4
    assert s1["AIME2025"]["metric"]["score_avg"] == pytest.approx(1 / 3)          # 0 right, 1 wrong, 2 failed
    assert s1["AIME2025"]["finish_reasons"] == {"stop": 2, "error": 1} and s1["IFBENCH"]["metric"]["score_avg"] == 1.0
    assert json.load(open(tmp_path / "out" / "summary.json")).keys() == s1.keys()
    cfg.eval()
    assert len(calls) == 4                                                          # everything came from the cache
    cfg.rerun_level = "error"
    s3 = cfg.eval()
    assert len(calls) == 5 and s3["AIME2025"]["metric"]["score_avg"] == pytest.approx(2 / 3)
    cfg.rerun_level, cfg.selected_datasets = "all", "IFBENCH"
    s4 = cfg.eval()
    assert list(s4) == ["IFBENCH"] and len(calls) == 6
    # decode limit fits the context: prompt of 3 tokens in a 100-token engine
    it = cfg.items_for(cfg.build_benchmarks()[0])[0]
    assert it.case.prompt.sampling_params.max_tokens == 96
    cfg.selected_datasets = "NOPE"
    with pytest.raises(ValueError):
        cfg.build_benchmarks()


def test_step3v_eval_samples_ifbench_four_times_at_temperature_one(tmp_path):
    from playground.eval.step3v.step3v_eval_simple_benchmarks import Exp
    from steptronoss_b200.exp.base_exp import TokenizerConfig

    (tmp_path / "IFBENCH").mkdir()
    (tmp_path / "IFBENCH" / "IFBench_test.jsonl").write_text(json.dumps(
        {"key": 1, "prompt": "no spaces please", "instruction_id_list": ["format:no_whitespace"], "kwargs": [{}]}))

    class Tok(TokenizerConfig):
        def build_tokenizer(self):
            return _Tok()

    exp = Exp()
    assert exp.resource_cfg.find_leaf_task_specs()["vllm"]["replica"] == 1 and exp.resource_cfg.gpu == 1
    assert exp.vllm_cfg.vllm_enforce_eager and exp.eval_cfg.tokenizer_cfg.tokenizer_path == exp.vllm_cfg.model_config_path
    exp._allow_set_new_attr = True
    exp.eval_cfg.tokenizer_cfg = Tok
    exp.eval_cfg.datasets_dir = str(tmp_path)
    (bench,) = exp.eval_cfg.build_benchmarks()
    cases = bench.get_cases()
    assert len(cases) == 4 and sorted(c.evaluation.run_index for c in cases) == [0, 1, 2, 3]
    sp = cases[0].prompt.sampling_params
    assert (sp.temperature, sp.top_p, sp.top_k) == (1.0, 1.0, 0)


def test_image_caption_data_feeds_the_vision_language_model(tmp_path):
    import numpy as np
    import torch
    from PIL import Image

    from playground.sft.step3v.image_caption_data import ImageCaptionDataConfig
    from steptronoss_b200.parallel.state import PM
    from tests.test_vl_model_cpu import _cfg

    for i in range(2):
        Image.fromarray((np.random.RandomState(i).rand(40, 50, 3) * 255).astype("uint8")).save(tmp_path / f"im{i}.png")
    (tmp_path / "captions.jsonl").write_text("\n".join(json.dumps({"image": f"im{i}.png", "caption": f"picture {i}"})
                                                        for i in range(2)))

    class ByteTok:
        def encode(self, text, add_special_tokens=False):
            return [4 + (b % 60) for b in text.encode()]

    class Data(ImageCaptionDataConfig):
        image_size, patch_size, img_start_token, image_token_id = 32, 4, 3, 2
        max_seq_len = 256

        def build_tokenizer(self):
            return ByteTok()

    d = Data()
    d.captions_file = str(tmp_path / "captions.jsonl")
    d.seqlen_divisible_by = 8
    stream = d.build_dataloader(dp_rank=1, dp_size=2)           # the second data-parallel rank starts at sample 1
    batch = next(stream)
    toks = batch["tokens"].tolist()
    assert toks.count(3) == 1 and toks.count(2) == d.features_per_image() == 4
    assert batch["images"].shape == (1, 3, 32, 32) and len(toks) % 8 == 0
    n_answer = len(ByteTok().encode("picture 1<|im_end|>\n"))
    assert int(batch["loss_mask"].sum()) == n_answer            # the loss covers the caption (shifted by one)
    assert stream.state_dict() == {"pos": 3}
    PM.initialize()
    cfg = _cfg()
    PM.set_mesh(cfg.parallel_cfg)
    model = cfg.build_model()
    model.init_weights(0, 0.02)
    feed = d.preprocess(batch)
    out = model(**{k: feed[k] for k in ("input_ids", "labels", "cu_seqlens", "max_seq_len", "images")},
                loss_masks=feed["loss_masks"])
    out["loss"].backward()
    assert torch.isfinite(out["loss"])
