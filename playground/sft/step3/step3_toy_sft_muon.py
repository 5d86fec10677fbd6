"""The Step-3.5 toy SFT run with Muon on the hidden matrices (reference
``playground/sft/step3/step3_toy_sft_step3_data_muon.py``)."""
from playground.sft.step3.muon_optimizer import MuonGradientManagerConfig
from playground.sft.step3.step3_toy_sft import Exp as AdamExp


class Exp(AdamExp):
    optimizer_cfg = MuonGradientManagerConfig


if __name__ == "__main__":
    Exp().train()
