"""Headline benchmark: Qwen3-8B dense training throughput (tokens/s over all GPUs of one node).

    python bench.py --gpus 1 --steps 3 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29500 \
        bench.py --gpus 8 --steps 3 --warmup 3

One step = one optimizer step over ``8 x N`` packed sequences of 8192 tokens (64 at 8 GPUs: weak
scaling), bf16 compute with fp32 master weights and Adam state, synthetic packed documents, random
N(0, 0.02) weights.  Two timed regions of K steps each, both bracketed by barrier + synchronize and
timed with CUDA events, max over ranks:

* ``value``: the training step with the step's micro-batches already resident on the device;
* ``e2e``: the same step through the public trainer API with every micro-batch copied from pinned
  host memory inside the timed region and the step loss read back to the host every step.

``--impl reference`` runs the unmodified reference framework (installed under ``baseline/_ref``) on
the same model/config through its own trainer, or reports why it cannot run.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# Wording shared by both arms, so that their JSON lines describe the same benchmark with the same `config`.
METRIC_TEXT = {"dense": "tokens/s/box (Qwen3-8B dense training, all GPUs of the node)",
               "moe": "tokens/s/box (Qwen3-30B-A3B-shape MoE pretraining, all GPUs of the node)"}
MODEL_TEXT = {"dense": "Qwen3-8B", "moe": "Qwen3-30B-A3B-shape MoE"}
DATA_TEXT = {"dense": "synthetic packed documents (lengths U[256,seq_len], uniform token ids), random N(0,0.02) init",
             "moe": "synthetic sequences of one document each (uniform token ids), random N(0,0.02) init"}
L2_TEXT = "inputs larger than L2 (each step streams > 100 GB)"


def scratch_dir() -> str:
    """Directory for the run's by-products (clock samples): ``STB200_BENCH_OUT`` or a temporary directory."""
    import tempfile

    d = os.environ.get("STB200_BENCH_OUT") or os.path.join(tempfile.gettempdir(), "stb200_bench")
    os.makedirs(d, exist_ok=True)
    return d


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="qwen3_8b", choices=["qwen3_8b", "qwen3_30b_a3b"],
                    help="qwen3_8b: the headline dense config; qwen3_30b_a3b: the MoE config (EP = N, attention DP = N, "
                         "sequences of 4096, 32 per GPU; its static state needs N >= 4)")
    ap.add_argument("--dispatcher", default="peer", choices=["peer", "alltoall"], help="MoE token dispatcher")
    ap.add_argument("--moe-capacity-factor", type=float, default=0.0,
                    help="MoE + peer dispatcher: size the expert buffers for this multiple of the balanced load instead "
                         "of reading the arrived count back every layer (0 = exact count, the default: the randomly "
                         "initialised 48-layer model on random tokens sends one rank more than twice its share at "
                         "EP=8, which a factor of 2 reports as the capacity error); overflow fails the run")
    ap.add_argument("--parallelism", default=None, help="e.g. tp4dp2, dp8, tp2, tp2cp2pp2; default tp=min(N,4) x dp")
    ap.add_argument("--optimizer", default="adam", choices=["adam", "muon"],
                    help="muon: Newton-Schulz updates for the 2-D hidden matrices, AdamW for the rest")
    ap.add_argument("--seqs-per-gpu", type=int, default=None,
                    help="sequences per GPU per step (global batch = this x N); default 8 (dense) / 32 (MoE)")
    ap.add_argument("--global-batch", type=int, default=None,
                    help="sequences per optimizer step of the whole job (overrides --seqs-per-gpu; e.g. 4 micro-batches "
                         "of one long sequence on a tp2cp2pp2 layout whose data-parallel degree is 1)")
    ap.add_argument("--seq-len", type=int, default=None, help="default 8192 (dense) / 4096 (MoE)")
    ap.add_argument("--seqs-per-micro-batch", type=int, default=1,
                    help="sequences packed into one forward/backward pass (as separate documents: attention, positions "
                         "and loss stay per sequence); the global batch and the tokens of a step do not change")
    ap.add_argument("--recompute", default="auto", help="auto | none | full | comma list of block parts")
    ap.add_argument("--recompute-layers", type=int, default=None,
                    help="recompute only the first N layers (default: 4 of 36 on one GPU, all otherwise)")
    ap.add_argument("--debug-layers", type=int, default=None, help="DEBUG ONLY: fewer layers (result marked invalid)")
    a = ap.parse_args()
    moe = a.model == "qwen3_30b_a3b"
    if a.seqs_per_gpu is None:
        a.seqs_per_gpu = 32 if moe else 8
    if a.seq_len is None:
        a.seq_len = 4096 if moe else 8192
    if a.seqs_per_micro_batch < 1 or a.seqs_per_gpu % a.seqs_per_micro_batch:
        ap.error("--seqs-per-micro-batch must divide the sequences per GPU")
    return a


class ClockSampler:
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, path, n_gpus=None):
        self.path, self.proc = path, None
        # sample only the GPUs this job runs on: an idle neighbour at its idle clock would skew the median
        n = int(n_gpus or os.environ.get("WORLD_SIZE", "1"))
        vis = [v for v in os.environ.get("CUDA_VISIBLE_DEVICES", "").split(",") if v.strip()]
        self.ids = vis[:n] if vis else [str(i) for i in range(n)]

    def start(self):
        try:
            self.f = open(self.path, "w")
            self.proc = subprocess.Popen(["nvidia-smi", "-i", ",".join(self.ids), f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "200"],
                                         stdout=self.f, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self, local_index=0):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.f.close()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in open(self.path):
            p = [x.strip() for x in line.split(",")]
            if len(p) < 9:
                continue
            try:
                sm.append(float(p[1]))
                mx.append(float(p[2]))
            except ValueError:
                continue
            for n, v in zip(names, p[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        busy = [s for s in sm if s > 0]
        return {"sm_mhz": statistics.median(busy) if busy else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


OPTIMIZER_TEXT = {"adam": "Adam fp32 master+state, ZeRO-1",
                  "muon": "Muon (2-D hidden matrices) + AdamW, fp32 master+state, ZeRO-1"}


def global_batch(args, world: int) -> int:
    return args.global_batch if args.global_batch else args.seqs_per_gpu * world


def default_parallelism(n: int) -> str:
    tp = min(n, 4)
    dp = n // tp
    return f"tp{tp}dp{dp}" if tp > 1 else f"dp{dp}"


def parse_parallelism(text: str) -> dict:
    import re

    out = {"tp": 1, "dp": 1, "pp": 1, "cp": 1, "ep": 1}
    for k, v in re.findall(r"([a-z]+)(\d+)", text):
        out[k] = int(v)
    return out


def model_flops_per_token(layers, hidden, heads, kv_heads, head_dim, ffn, vocab, avg_ctx, router_experts=0):
    """``ffn`` is the SwiGLU width a token passes through (top-k x expert width for a routed FFN)."""
    qkv = hidden * (heads + 2 * kv_heads) * head_dim
    o = heads * head_dim * hidden
    mlp = 3 * hidden * ffn + hidden * router_experts
    dense = layers * (qkv + o + mlp) + vocab * hidden
    attn = layers * 2 * heads * head_dim * avg_ctx  # QK^T and PV, causal average context
    return 6 * dense + 6 * attn


def run_ours(args):
    import torch
    import torch.distributed as dist

    moe = args.model == "qwen3_30b_a3b"
    if moe:
        from playground.pretrain.qwen3.qwen3_30a3b import Exp
    else:
        from playground.pretrain.qwen3.qwen3_8b import Exp
    from steptronoss_b200.ops import launch_count
    from steptronoss_b200.ops import native

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}; launch with torch.distributed.run for N>1")
    par_text = args.parallelism or (f"ep{world}dp{world}" if moe else default_parallelism(world))
    par = parse_parallelism(par_text)
    exp = Exp()
    pc = exp.model_cfg.parallel_cfg
    if moe:
        pc.expert_model_parallel_size, pc.expert_tensor_parallel_size = par["ep"], 1
        exp.model_cfg.moe_cfg.dispatcher = args.dispatcher
        exp.model_cfg.moe_cfg.capacity_factor = args.moe_capacity_factor or None
        if args.debug_layers:
            exp.model_cfg.moe_cfg.moe_layer_list = list(range(args.debug_layers))
    pc.tensor_model_parallel_size = par["tp"]
    pc.pipeline_model_parallel_size = par["pp"]
    pc.context_parallel_size = par["cp"]
    exp.model_cfg.tp_cfg.sequence_parallel = par["tp"] > 1
    if args.optimizer == "muon":
        from steptronoss_b200.exp.optimizer import MuonConfig

        exp.optimizer_cfg.optimizer_cfg = MuonConfig
    tc = exp.trainer_cfg
    # a micro-batch of M sequences is one packed row of M x seq_len tokens whose documents are at most seq_len long
    tc.global_seq_length = args.seq_len * args.seqs_per_micro_batch
    tc.global_batch_size = global_batch(args, world) // args.seqs_per_micro_batch
    tc.train_iters = 10**9
    tc.writer_backend = []
    tc.log_interval = 10**9
    exp.data_cfg.max_doc_len = args.seq_len
    if moe:
        exp.data_cfg.min_doc_len = args.seq_len  # one document per sequence
    if args.debug_layers:
        exp.model_cfg.num_layers = args.debug_layers
    rec = args.recompute
    if rec == "auto":
        # one GPU holds 18 bytes/parameter of static state (147 GB): recompute whole blocks
        rec = "full" if par["tp"] * par["pp"] == 1 and not moe else "none"
    exp.model_cfg.recompute = True if rec == "full" else ([] if rec == "none" else rec.split(","))
    rec_layers = args.recompute_layers
    if rec_layers is None and rec == "full" and args.recompute == "auto" and not args.debug_layers:
        rec_layers = 4  # 147 GB of static state + the activations of 32 layers peak near 168 GB of the 179 GB
    if rec_layers is not None:
        exp.model_cfg.recompute_num_layers = rec_layers
        rec = f"{rec} (first {rec_layers} layers)"
    exp.resource_cfg.gpu = world
    os.environ.setdefault("WORLD_SIZE", str(world))
    os.environ.setdefault("STEPTRON_QUIET_EXP", "1")     # the config tree is not part of a benchmark log
    exp.sanity_check()
    trainer = exp.trainer_cfg.get_trainer_cls()(exp=exp)
    trainer.before_train()
    dev = trainer.device

    def barrier_sync():
        if dist.is_initialized():
            dist.barrier()
        torch.cuda.synchronize()

    from steptronoss_b200.utils.metrics import GlobalMetrics

    loss_step0 = None
    for w in range(args.warmup):
        trainer.train_step()
        if w == 0:
            # Loss of the first micro-batch of the first step, before any update.  Rank 0's first sample is the same
            # in every layout and the initial weights do not depend on the layout, so this number must agree
            # across N = 1, 2, 4, 8 to bf16 rounding.
            vals = GlobalMetrics.metrics["lm_loss"].values if "lm_loss" in GlobalMetrics.metrics else []
            if vals:
                first = torch.as_tensor(vals[0]).float().mean().to(dev)
                if par["cp"] > 1:   # a CP rank holds the sum over its own tokens divided by the count of all tokens
                    from steptronoss_b200.parallel.state import PM

                    dist.all_reduce(first, group=PM.group_of("CP"))
                loss_step0 = float(first.item())
    barrier_sync()
    native.raise_if_kernel_error()

    n_micro = trainer.num_microbatches()
    tokens_per_step = tc.global_batch_size * tc.global_seq_length

    # ---- region A: device-resident inputs --------------------------------------------------------
    class Staged:
        def __init__(self, src, count):
            self.items = []
            if src is not None:
                for _ in range(count):
                    self.items.append({k: v.to(dev) for k, v in next(src).items()})
            self.pos = 0

        def __iter__(self):
            return self

        def __next__(self):
            x = self.items[self.pos]
            self.pos += 1
            return x

    live_iters = trainer.data_iterators
    staged = [Staged(it, n_micro * args.steps) for it in live_iters]
    trainer.data_iterators = [s if it is not None else None for s, it in zip(staged, live_iters)]
    sampler = ClockSampler(os.path.join(scratch_dir(), "bench_clocks.csv"), world) if rank == 0 else None
    if sampler:
        sampler.start()
    barrier_sync()
    l0 = launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        trainer.train_step()
    e1.record()
    barrier_sync()
    launches = launch_count() - l0
    ms_a = e0.elapsed_time(e1)
    clocks = sampler.stop() if sampler else None
    trainer.data_iterators = live_iters

    # ---- region B: end to end (pinned host inputs copied in, loss read back every step) ----------
    h2d = d2h = 0
    for s_ in staged:
        if s_.items:
            h2d = sum(v.numel() * v.element_size() for v in s_.items[0].values()) * n_micro
            break
    barrier_sync()
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    f0.record()
    last_loss = None
    for _ in range(args.steps):
        trainer.train_step()
        vals = GlobalMetrics.metrics["lm_loss"].values
        if vals:
            last_loss = float(torch.stack([torch.as_tensor(v) for v in vals]).mean().item())  # D2H read
            d2h = 4
        GlobalMetrics.reset()
    f1.record()
    barrier_sync()
    wall_b = (time.perf_counter() - t0) * 1e3
    ms_b = max(f0.elapsed_time(f1), wall_b)
    native.raise_if_kernel_error()

    t = torch.tensor([ms_a, ms_b], dtype=torch.float64, device=dev)
    if dist.is_initialized():
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_a, ms_b = float(t[0]), float(t[1])
    if rank != 0:
        return
    value = tokens_per_step * args.steps / (ms_a / 1e3)
    e2e = tokens_per_step * args.steps / (ms_b / 1e3)
    mc = exp.model_cfg
    avg_ctx = (args.seq_len ** 2 / 3.0) / ((256 + args.seq_len) / 2.0) / 2.0 if args.seq_len > 256 else args.seq_len / 2
    if moe:
        avg_ctx = args.seq_len / 2.0  # one document per sequence
        fpt = model_flops_per_token(mc.num_layers, 2048, 32, 4, 128, 8 * 768, 151936, avg_ctx, router_experts=128)
    else:
        fpt = model_flops_per_token(mc.num_layers, 4096, 32, 8, 128, 12288, 151936, avg_ctx)
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except Exception:
        pass
    peak = float(peaks.get("bf16_tflops_sustained", 1375.7)) * 1e12
    kind = "moe" if moe else "dense"
    out = {
        "metric": METRIC_TEXT[kind],
        "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_a / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16",
        "data": DATA_TEXT[kind],
        "mfu_of_measured_sustained_bf16": value * fpt / (peak * world),
        "config": {"model": MODEL_TEXT[kind], "layers": mc.num_layers, "global_batch": global_batch(args, world),
                   "seq_len": args.seq_len, "micro_batch": args.seqs_per_micro_batch, "parallelism": par_text,
                   "optimizer": OPTIMIZER_TEXT[args.optimizer], "recompute": rec, "l2": L2_TEXT},
        "implementation": {"attention": "tcgen05 flash attention (csrc/attention_sm100.cu)",
                           **({"moe_dispatcher": args.dispatcher,
                               "moe_capacity_factor": args.moe_capacity_factor or None} if moe else {})},
        "clocks": clocks,
        "loss_step0": loss_step0,
        "e2e": {"value": e2e, "unit": "tokens/s", "ms_per_step": ms_b / args.steps, "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h, "last_loss": last_loss},
        "gpu_launches": launches,
        "peak_memory_gb": torch.cuda.max_memory_allocated() / 2 ** 30,
        "impl": "ours",
    }
    if args.debug_layers:
        out["invalid_debug_config"] = True
    print(json.dumps(out), flush=True)


def run_reference(args):
    sys.path.insert(0, os.path.join(ROOT, "baseline"))
    try:
        from reference_arm import run as ref_run
    except Exception as e:  # the arm is optional: report instead of failing
        print(json.dumps({"impl": "reference", "unavailable": f"reference arm not importable: {type(e).__name__}: {e}"}))
        return
    ref_run(args)


if __name__ == "__main__":
    import faulthandler

    faulthandler.enable()
    # a run that exceeds this many seconds (a rank lost in a collective after another one failed) dumps every
    # thread's stack and exits instead of waiting for the process-group timeout; 0 switches the limit off
    limit = int(os.environ.get("STB200_BENCH_WATCHDOG_S", "1800"))
    if limit > 0:
        faulthandler.dump_traceback_later(limit, exit=True)
    a = parse()
    if a.impl == "reference":
        run_reference(a)
    else:
        try:
            run_ours(a)
        except BaseException:
            if int(os.environ.get("WORLD_SIZE", "1")) > 1 and not isinstance(sys.exc_info()[1], SystemExit):
                # the other ranks may sit in a collective waiting for this one: show why and end the job now
                import traceback

                traceback.print_exc()
                sys.stderr.flush()
                os._exit(1)
            raise
