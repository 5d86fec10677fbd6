"""Two SFT steps of Step3-VL-10B on image-caption pairs under TP=8: a smoke run of the whole vision-language path
(HF weights in, vision encoder, feature insertion, tensor-parallel text stack, one optimizer step) (reference
``playground/sft/step3v/step3v_10b_sft_tp8_flickr8k_smoke.py``).

    python -m steptronoss_b200.launch.mp_run playground/sft/step3v/step3v_10b_sft_tp8_caption_smoke.py \\
        data_cfg.captions_file=/data/flickr8k/captions.jsonl checkpoint_cfg.load_safetensors=/models/Step3-VL-10B
"""
from playground.pretrain.step3v.step3v_10b import Step3V10BConfig
from playground.sft.qwen3.qwen3_sft_base import Exp as BaseExp
from playground.sft.step3v.image_caption_data import ImageCaptionDataConfig
from steptronoss_b200.exp.base_exp import TokenizerConfig


class Exp(BaseExp):
    model_cfg = Step3V10BConfig
    data_cfg = ImageCaptionDataConfig
    tokenizer_cfg: TokenizerConfig = TokenizerConfig

    def __init__(self):
        super().__init__()
        t = self.trainer_cfg
        t.micro_batch_size, t.global_batch_size = 1, 1
        t.global_seq_length = self.data_cfg.max_seq_len
        t.train_iters, t.log_interval = 2, 1
        s = self.scheduler_cfg
        s.warmup_schedule, s.lr, s.weight_decay = 0, 1e-5, 0.0
        m = self.model_cfg
        m.recompute = True
        m.tp_cfg.sequence_parallel = False      # image features are spliced in before the sequence is scattered
        m.parallel_cfg.tensor_model_parallel_size = 8
        m.tok_embed_cfg.encoder_cfg.parallel_cfg.tensor_model_parallel_size = 8
        c = self.checkpoint_cfg
        c.load_option.none(but=["model"])
        c.save_option.none()
        c.save_safetensors, c.save_interval, c.auto_resume = False, None, False
        self.profiler_cfg.timing_log_level = 1


if __name__ == "__main__":
    Exp().train()
