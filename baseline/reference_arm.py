"""Baseline arm of ``bench.py``: the unmodified reference framework training the same model.

The reference tree is copied verbatim to ``baseline/_ref`` (it is pure Python; its own build backend,
hatchling, is not installable offline) and imported from there.  Two of its dependencies are not
installable either and are replaced by the small stand-ins under ``baseline/shims``:
``configurize`` (mapped to this repository's implementation of the same config-tree API) and
``megfile`` (local file system).  Everything on the training path — models, tensor-parallel layers,
flash-attn attention core, MoE block with its all-to-all ``TokenDispatcher`` and grouped GEMM, gradient
manager, optimizer, schedule, trainer — is the reference's own code, driven through its own ``Exp`` /
trainer API with its own configuration files (``playground/pretrain/qwen3/qwen3_8b.py`` for the dense
model, ``playground/pretrain/qwen3/qwen3_30a3b.py`` for the MoE model).

The MoE arm selects, through the reference's own ``set_optimization`` switch, the fastest alternatives the
reference ships that can run here: flash-attn attention, its Triton grouped GEMM (the ``grouped_gemm`` wheel
and DeepEP are not installed) and its Triton routing / scatter / gather kernels.
``STB200_REF_GROUPED_GEMM`` (``triton_grouped_gemm`` | ``function_imple`` | ``default``) and
``STB200_REF_MOE_TRITON=0`` choose the slower statements instead.

Only two things are supplied from outside, because the reference does not ship them: a synthetic
packed-document data config producing the reference's batch contract, and a weight initialiser
(the reference leaves parameters uninitialised and expects a checkpoint).
"""
from __future__ import annotations

import importlib.util
import json
import os
import sys
import time
import traceback

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")


def _load_file(path: str, name: str):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


def _scratch_dir() -> str:
    """Where the run's own by-products (clock samples, the reference's log directory) go."""
    import tempfile

    d = os.environ.get("STB200_BENCH_OUT") or os.path.join(tempfile.gettempdir(), "stb200_bench")
    os.makedirs(d, exist_ok=True)
    return d


def _unavailable(why: str, any_rank: bool = False):
    if any_rank or int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps({"impl": "reference", "unavailable": why.replace("\n", " ")[:400]}), flush=True)


def run(args) -> None:
    if not os.path.isdir(os.path.join(REF, "steptronoss")):
        return _unavailable("baseline/_ref/steptronoss is absent: copy the reference tree there first")
    sys.path.insert(0, os.path.join(HERE, "shims"))
    sys.path.insert(0, REF)
    try:
        _run(args)
    except BaseException as e:  # report instead of failing the driver
        sys.stderr.write(traceback.format_exc())
        tb = traceback.format_exc().strip().splitlines()
        world = int(os.environ.get("WORLD_SIZE", "1"))
        # the rank that failed reports (the others may be waiting for it inside a collective and never will)
        _unavailable(f"rank {os.environ.get('RANK', '0')}: {type(e).__name__}: {e} | {tb[-3] if len(tb) > 3 else ''}",
                     any_rank=world > 1)
        if world > 1:
            # end the whole job now: a clean return would leave the other ranks in their collective until the
            # process-group timeout; the launcher stops them when one worker exits with an error
            sys.stdout.flush()
            os._exit(3)


def _run(args) -> None:
    import numpy as np
    import torch
    import torch.distributed as dist

    os.environ.setdefault("CUDA_DEVICE_MAX_CONNECTIONS", "1")
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    os.environ.setdefault("WORLD_SIZE", "1")
    os.environ.setdefault("RANK", "0")
    os.environ.setdefault("LOCAL_RANK", "0")
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29533")

    from steptronoss.exp.base_exp import DataConfig
    from steptronoss.core.trainers.lm_trainer import DecoderPretrainTrainer

    moe = getattr(args, "model", "qwen3_8b") == "qwen3_30b_a3b"
    sft_base = _load_file(os.path.join(REF, "playground/sft/qwen3/qwen3_sft_base.py"), "_ref_qwen3_sft_base")
    if moe:
        model_file = _load_file(os.path.join(REF, "playground/pretrain/qwen3/qwen3_30a3b.py"), "_ref_qwen3_30a3b")
        model_cfg_cls = model_file.Qwen3_30A3BConfig
    else:
        model_file = _load_file(os.path.join(REF, "playground/pretrain/qwen3/qwen3_8b.py"), "_ref_qwen3_8b")
        model_cfg_cls = model_file.Qwen3_8BConfig

    sys.path.insert(0, os.path.dirname(HERE))
    from bench import OPTIMIZER_TEXT, ClockSampler, default_parallelism, global_batch, model_flops_per_token, parse_parallelism
    from steptronoss_b200.data.synthetic import make_packed_sample  # data generator only (numpy)

    par_text = args.parallelism or (f"ep{world}dp{world}" if moe else default_parallelism(world))
    par = parse_parallelism(par_text)
    seq = args.seq_len
    min_doc = seq if moe else 256          # the MoE config trains on one document per sequence

    class Loader:
        def __init__(self, dp_rank, dp_size):
            self.i, self.dp_rank, self.dp_size = 0, dp_rank, dp_size

        def __iter__(self):
            return self

        def __len__(self):
            return 1 << 40

        def __next__(self):
            rng = np.random.default_rng([0, self.i * self.dp_size + self.dp_rank])
            self.i += 1
            s = make_packed_sample(rng, seq, 151936, min_doc, seq)
            return {k: v.pin_memory() for k, v in s.items()}

        def state_dict(self):
            return {"i": self.i}

        def load_state_dict(self, sd):
            self.i = sd["i"]

    class SyntheticData(DataConfig):
        global_data_keys = ["cu_seqlens", "position_id", "max_seq_len"]

        def build_dataloader(self, dp_rank=0, dp_size=1):
            return Loader(dp_rank, dp_size)

    class Trainer(DecoderPretrainTrainer):
        def setup_model(self, model_config):
            models = super().setup_model(model_config)
            gen = torch.Generator(device="cuda")
            gen.manual_seed(1234 + rank)
            with torch.no_grad():
                for m in models:
                    for n, p in m.named_parameters():
                        if p.dim() == 1:
                            p.fill_(1.0)
                        else:
                            p.normal_(0.0, 0.02, generator=gen)
            return models

    moe_choices = {}

    class Exp(sft_base.Exp):
        model_cfg = model_cfg_cls
        data_cfg = SyntheticData

        def __init__(self):
            super().__init__()
            pc = self.model_cfg.parallel_cfg
            pc.tensor_model_parallel_size = par["tp"]
            pc.pipeline_model_parallel_size = par["pp"]
            pc.context_parallel_size = par["cp"]
            self.model_cfg.tp_cfg.sequence_parallel = par["tp"] > 1
            self.model_cfg.check_nan = False
            if args.optimizer == "muon":
                from steptronoss.exp.optimizer import MuonConfig as RefMuonConfig

                self.optimizer_cfg.optimizer_cfg = RefMuonConfig
            if moe:
                pc.expert_model_parallel_size, pc.expert_tensor_parallel_size = par["ep"], 1
                self.model_cfg.ffn_cfg.moe_cfg.moe_aux_loss_coef = 1e-3
            if args.debug_layers:
                self.model_cfg.num_layers = args.debug_layers
                if moe:
                    self.model_cfg.ffn_cfg.moe_cfg.moe_layer_list = list(range(args.debug_layers))
            rec = args.recompute
            if rec == "auto":
                rec = "full" if par["tp"] * par["pp"] == 1 and not moe else "none"
            self.model_cfg.recompute = True if rec == "full" else ([] if rec == "none" else rec.split(","))
            self._recompute_text = rec
            t = self.trainer_cfg
            t.global_batch_size = global_batch(args, world)
            t.global_seq_length = seq
            t.micro_batch_size = 1
            t.train_iters = 10 ** 9
            t.log_interval = 10 ** 9
            self.resource_cfg.gpu = world
            self.scheduler_cfg.lr = 1e-5
            self.scheduler_cfg.weight_decay = 0.1
            self.scheduler_cfg.total_schedule = 10 ** 6
            self.scheduler_cfg.warmup_schedule = 0
            self.checkpoint_cfg.save_interval = None
            self.log_dir = os.path.join(_scratch_dir(), "reference_logs")

        def configure_optimizable(self):
            if not moe:
                return super().configure_optimizable()    # the reference's own choice for its dense experiments
            from steptronoss.utils.optimizable import set_optimization

            gg = os.environ.get("STB200_REF_GROUPED_GEMM", "triton_grouped_gemm")
            kw = {"AttentionCore": "flash-attn"}
            if gg != "default":
                kw["grouped_gemm"] = gg
            if os.environ.get("STB200_REF_MOE_TRITON", "1") != "0":
                kw.update(histogram="triton", index_compute="triton", moe_scatter="triton", moe_weighted_gather="triton")
            set_optimization(**kw)
            moe_choices.update(kw)

    exp = Exp()
    exp.sanity_check()
    os.environ["WORLD_SIZE"] = str(world)
    trainer = Trainer(exp=exp)
    exp.configure_optimizable()  # dense: the reference experiment's own choice (flash-attn core, torch.compile default)
    trainer.before_train()
    for m in trainer.models:
        m.train()
    trainer.iteration = 0

    def barrier_sync():
        if dist.is_initialized():
            dist.barrier()
        torch.cuda.synchronize()

    def step():
        trainer.train_step()
        trainer.iteration += 1

    for _ in range(args.warmup):
        step()
    barrier_sync()
    sampler = ClockSampler(os.path.join(_scratch_dir(), "bench_clocks_reference.csv"), world) if rank == 0 else None
    if sampler:
        sampler.start()
    barrier_sync()
    # STB200_REF_CPROFILE=1: run the timed steps under cProfile on rank 0 and report which share of the host time
    # is spent inside the stand-in for `configurize` (this repository's config tree), i.e. how much the stand-in
    # could distort the reference's number.  Off by default: profiling slows the host down.
    profiler = None
    if os.environ.get("STB200_REF_CPROFILE") == "1" and rank == 0:
        import cProfile

        profiler = cProfile.Profile()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    e0.record()
    if profiler is not None:
        profiler.enable()
    for _ in range(args.steps):
        step()
    if profiler is not None:
        profiler.disable()
    e1.record()
    barrier_sync()
    wall = (time.perf_counter() - t0) * 1e3
    ms = e0.elapsed_time(e1)
    shim_share = None
    if profiler is not None:
        import pstats

        stats = pstats.Stats(profiler)
        total = sum(v[2] for v in stats.stats.values())                       # tottime over all functions
        in_shim = sum(v[2] for (fname, _, _), v in stats.stats.items()
                      if "steptronoss_b200/config/" in fname.replace(os.sep, "/") or "/shims/configurize/" in fname.replace(os.sep, "/"))
        shim_share = {"host_seconds_profiled": total, "seconds_in_config_stand_in": in_shim,
                      "share": in_shim / total if total else 0.0}
    clocks = sampler.stop() if sampler else None
    t = torch.tensor([ms, wall], dtype=torch.float64, device="cuda")
    if dist.is_initialized():
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, wall = float(t[0]), float(t[1])
    if rank != 0:
        return
    tc = exp.trainer_cfg
    tokens = tc.global_batch_size * tc.global_seq_length
    value = tokens * args.steps / (ms / 1e3)
    # the reference's step already copies every micro-batch from pinned host memory and reads the loss,
    # the gradient norm and a NaN flag back to the host, so its end-to-end figure is the same run
    e2e = tokens * args.steps / (max(ms, wall) / 1e3)
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(os.path.dirname(HERE), "MEASURED_PEAKS.json")))
    except Exception:
        pass
    peak = float(peaks.get("bf16_tflops_sustained", 1375.7)) * 1e12
    if moe:
        fpt = model_flops_per_token(exp.model_cfg.num_layers, 2048, 32, 4, 128, 8 * 768, 151936, seq / 2.0,
                                    router_experts=128)
    else:
        avg_ctx = (seq ** 2 / 3.0) / ((256 + seq) / 2.0) / 2.0
        fpt = model_flops_per_token(exp.model_cfg.num_layers, 4096, 32, 8, 128, 12288, 151936, avg_ctx)
    from bench import DATA_TEXT, L2_TEXT, METRIC_TEXT, MODEL_TEXT

    kind = "moe" if moe else "dense"
    out = {
        "metric": METRIC_TEXT[kind], "value": value, "unit": "tokens/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": DATA_TEXT[kind],
        "mfu_of_measured_sustained_bf16": value * fpt / (peak * world),
        # the same keys, in the same words, as the other arm prints
        "config": {"model": MODEL_TEXT[kind], "layers": exp.model_cfg.num_layers, "global_batch": tc.global_batch_size,
                   "seq_len": seq, "micro_batch": 1, "parallelism": par_text, "optimizer": OPTIMIZER_TEXT[args.optimizer],
                   "recompute": exp._recompute_text, "l2": L2_TEXT},
        "implementation": {"attention": "flash-attn 2 (reference AttentionCore)",
                           **({"moe_dispatcher": "TokenDispatcher (NCCL all-to-all)", "optimizable": moe_choices}
                              if moe else {"optimizable": "AttentionCore=flash-attn, default=torch_compile"})},
        "clocks": clocks,
        "e2e": {"value": e2e, "unit": "tokens/s", "ms_per_step": max(ms, wall) / args.steps},
        "impl": "reference",
    }
    if shim_share is not None:
        out["config_stand_in_profile"] = shim_share
        out["invalid_profiled_run"] = True      # a number taken under a profiler is not a benchmark value
    if args.debug_layers:
        out["invalid_debug_config"] = True
    print(json.dumps(out), flush=True)
