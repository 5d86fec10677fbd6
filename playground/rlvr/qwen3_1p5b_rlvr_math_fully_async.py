"""The RLVR math run under fully asynchronous flow control (reference
``playground/rlvr/qwen3_1p5b_rlvr_math_fully_async.py``): generation never waits for a training step as long as
at most ``max_untrained_prompts`` prompts are outstanding and no running prompt would fall more than
``max_staleness`` weight versions behind; a step starts as soon as ``prompt_per_iter`` prompts have finished.
``python -m steptronoss_b200.generators.flow_controller_simulator`` shows the timeline such settings give.
"""
from playground.rlvr.qwen3_1p5b_rlvr_math import Exp as BaseExp
from playground.rlvr.qwen3_1p5b_rlvr_math import RLVRTrainerConfig
from steptronoss_b200.exp.rl import FullyAsyncFlowControllerConfig


class FullyAsyncMathFlowControllerConfig(FullyAsyncFlowControllerConfig):
    def __init__(self):
        super().__init__()
        self.prompt_per_iter = 16
        self.max_untrained_prompts = 32
        self.max_staleness = 2


class FullyAsyncRLVRTrainerConfig(RLVRTrainerConfig):
    flow_cfg = FullyAsyncMathFlowControllerConfig


class Exp(BaseExp):
    trainer_cfg = FullyAsyncRLVRTrainerConfig

    def __init__(self):
        super().__init__()
        self.checkpoint_cfg.save_dir = "./checkpoints_fully_async"


if __name__ == "__main__":
    Exp().entrypoint()
