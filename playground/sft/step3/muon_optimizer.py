"""Muon settings of the Step-3.5 SFT runs (reference ``playground/sft/step3/muon_optimizer.py``): weight decay
also on 1-D parameters, six Newton-Schulz steps with the polar-express coefficients, stacked expert weights
treated as one matrix per expert, embeddings and the LM head on the AdamW branch."""
from steptronoss_b200.exp.base_exp import GradientManagerConfig
from steptronoss_b200.exp.optimizer import MuonConfig


class Step3p5MuonConfig(MuonConfig):
    def __init__(self):
        super().__init__()
        self.weight_decay_on_1d_params = True
        self.muon_ns_steps = 6
        self.muon_newtonschulz_fn = "polar_express"
        self.muon_min_ndim_is_2_only = False


class MuonGradientManagerConfig(GradientManagerConfig):
    optimizer_cfg = Step3p5MuonConfig
