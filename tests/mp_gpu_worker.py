"""Worker for the multi-GPU tests: trains the tiny bf16 experiment under the layout given on the command
line (launched by torch.distributed.run) and prints one JSON line with the loss curve from rank 0.
With ``cpu_fp32`` as third argument it trains the same experiment in fp32 through the PyTorch restatements
(the caller hides the GPUs): the oracle of the single-GPU end-to-end test."""
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402


def main():
    kw = json.loads(sys.argv[1])
    steps = int(sys.argv[2])
    from steptronoss_b200.ops import native
    from steptronoss_b200.parallel.state import PM
    from tests.tiny_exp import make_tiny_exp

    PM.initialize()
    cpu_oracle = len(sys.argv) > 3 and sys.argv[3] == "cpu_fp32"
    exp = make_tiny_exp(dtype=torch.float32 if cpu_oracle else torch.bfloat16, **kw)
    exp.seed = 0
    tr = exp.trainer_cfg.get_trainer_cls()(exp=exp)
    tr.before_train()
    losses = []
    for _ in range(steps):
        tr.train_step()
        tr.iteration += 1
        tr.training_log()
        losses.append(tr.history[-1]["lm_loss"])
    if torch.cuda.is_available():
        torch.cuda.synchronize()
        native.raise_if_kernel_error()
    if PM.world_rank == PM.world_size - 1:
        gm = getattr(tr, "grad_manager", None) or getattr(tr, "gm", None)
        print("RESULT " + json.dumps({"losses": losses, "grad_norms": [h["grad_norm"] for h in tr.history],
                                      "peer_zero_groups": sorted(getattr(gm, "_peer", {}) or {})}), flush=True)
    if torch.distributed.is_initialized():
        torch.distributed.barrier()


if __name__ == "__main__":
    main()
