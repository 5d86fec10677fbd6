"""Run every kernel micro-benchmark and collect their JSON rows in one directory (the reference's
``benchmarks/run_all.sh``).  Single-GPU benchmarks run as they are; the multi-rank ones are started through
``torch.distributed.run`` on ``--gpus`` GPUs when more than one is visible.

    python benchmarks/run_all.py [--out bench_out] [--gpus 8] [--skip attention,zero]
"""
from __future__ import annotations

import argparse
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
SINGLE = {"gemm": ["benchmark_gemm.py"], "fp8_gemm": ["benchmark_fp8_gemm.py"], "attention": ["benchmark_attention.py"],
          "moe": ["benchmark_moe.py"], "muon": ["benchmark_muon.py"]}
# the multi-rank ones need at least two GPUs, except the MoE layer (which then runs its single-rank variant)
MULTI = {"moe_layer": ["benchmark_moe_layer.py"], "zero": ["benchmark_zero_peer.py"], "fused_tp": ["benchmark_fused_tp.py"],
         "cp_attention": ["benchmark_cp_attention.py"], "peer_bandwidth": ["benchmark_peer_bandwidth.py", "--no-ring"]}


def commands(out: str, gpus: int, skip: set) -> list:
    cmds = []
    for name, (script, *rest) in SINGLE.items():
        if name in skip:
            continue
        extra = [] if name == "attention" else ["--json", os.path.join(out, f"{name}.json")]
        cmds.append((name, [sys.executable, os.path.join(HERE, script), *rest, *extra]))
    for name, (script, *rest) in MULTI.items():
        if name in skip or (name != "moe_layer" and gpus < 2):
            continue
        launcher = ([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={gpus}",
                     "--master-addr", "127.0.0.1", "--master-port", "29871"] if gpus > 1 else [sys.executable])
        cmds.append((name, [*launcher, os.path.join(HERE, script), *rest, "--json", os.path.join(out, f"{name}.json")]))
    return cmds


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default="bench_out")
    ap.add_argument("--gpus", type=int, default=None)
    ap.add_argument("--skip", default="")
    ap.add_argument("--dry-run", action="store_true", help="print the commands only")
    a = ap.parse_args(argv)
    gpus = a.gpus
    if gpus is None:
        import torch

        gpus = max(torch.cuda.device_count(), 1)
    os.makedirs(a.out, exist_ok=True)
    failed = []
    for name, cmd in commands(a.out, gpus, {s for s in a.skip.split(",") if s}):
        print("+ " + " ".join(cmd), flush=True)
        if a.dry_run:
            continue
        with open(os.path.join(a.out, f"{name}.log"), "w") as log:
            rc = subprocess.call(cmd, stdout=log, stderr=subprocess.STDOUT)
        print(f"  {name}: exit {rc}", flush=True)
        if rc:
            failed.append(name)
    return 1 if failed else 0


if __name__ == "__main__":
    raise SystemExit(main())
