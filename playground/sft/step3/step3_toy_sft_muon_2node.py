"""Two nodes of 8 GPUs: the toy Muon SFT run with data parallelism across the nodes (reference
``playground/sft/step3/step3_toy_sft_step3_data_muon_2node.py``)."""
from playground.sft.step3.step3_toy_sft_muon import Exp as OneNodeExp


class Exp(OneNodeExp):
    def __init__(self):
        super().__init__()
        self.resource_cfg.replica = 2
        self.trainer_cfg.global_batch_size = 16


if __name__ == "__main__":
    Exp().train()
