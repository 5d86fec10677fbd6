"""Experiment-level configuration tree (reference ``steptronoss/exp/base_exp.py:39-519``).

Field names follow the reference so that experiment files port by changing the import root.
"""
from __future__ import annotations

import inspect
import os
from functools import cached_property
from typing import Any

import torch

from ..config import Config, Ref, parse_args, writable_property
from .abstract import DataConfig as AbstractDataConfig
from .abstract import MetricConfig as AbstractMetricConfig
from .abstract import ModelConfig as AbstractModelConfig
from .abstract import TokenizerConfig as AbstractTokenizerConfig
from .abstract import TrainerConfig as AbstractTrainerConfig
from .optimizer import AdamConfig, OptimizerConfig
from .resources import ResourceConfig


def is_log_rank() -> bool:
    return int(os.getenv("RANK", "0")) == 0


class GradientManagerConfig(Config):
    optimizer_cfg: OptimizerConfig = AdamConfig
    params_dtype = Ref("..model_cfg.params_dtype", torch.bfloat16)
    use_distributed_optimizer: bool = True
    clip_grad: float = 1.0
    log_detailed_grad_norms: bool = Ref("..trainer_cfg.log_detailed_grad_norms", False)
    log_num_zeros_in_grad: bool = Ref("..trainer_cfg.log_num_zeros_in_grad", False)
    overlap_param_gather: bool = True
    """Issue the bf16 parameter all-gather of the next step on a side stream right after the
    optimizer update instead of blocking (no reference counterpart)."""

    def build_gradient_manager(self, model):
        from ..optim.gradient_manager import AccInFP32GradientManager, DummyOptimizer, Zero1GradientManager

        models = model if isinstance(model, (list, tuple)) else [model]
        if not any(p.requires_grad for m in models for p in m.parameters()):
            return DummyOptimizer()
        cls = Zero1GradientManager if self.use_distributed_optimizer else AccInFP32GradientManager
        return cls(cfg=self, model=model)


class MetricConfig(AbstractMetricConfig):
    _allow_set_new_attr = True

    def register(self) -> None:
        from ..utils.metrics import GlobalMetrics

        self.register_metric()
        GlobalMetrics.batch_register(self)

    def __init__(self) -> None:
        super().__init__()
        from ..utils.metrics import GradNormMetric, Metric

        self.consumed_tokens = Metric().sum("time").sum("dp")
        self.iteration_time = Metric().mean("time")
        self.learning_rate = Metric().mean("time")
        self.grad_norms = GradNormMetric()


class TrainerConfig(AbstractTrainerConfig):
    micro_batch_size: int = 1
    global_batch_size: int = 8
    global_seq_length: int = 8192
    train_iters: int | None = None
    offload_optimizer_state: bool = False
    global_data_keys = Ref("..data_cfg.global_data_keys", None)
    empty_unused_memory_level: int = 0
    log_detailed_grad_norms: bool = False
    log_num_zeros_in_grad: bool = False
    log_interval: int = 1
    writer_backend: list = ["tensorboard"]
    model_cfg = Ref("..model_cfg", None)
    data_cfg = Ref("..data_cfg", None)

    # ---- hook points: each returns a list of ``fn(trainer)``; override in an experiment's trainer config -----------
    def build_after_init_hooks(self) -> list:
        """Run once the process group, the mesh and the metrics exist, before any model is built.  By default the
        log rank prints the resolved experiment tree, so that a job's log says what was run."""

        def print_exp(trainer):
            from ..utils.logger import logger

            if int(os.getenv("RANK", "0")) == 0 and not os.getenv("STEPTRON_QUIET_EXP"):
                try:
                    logger.info(f"experiment:\n{self.root()}", at=None)
                except Exception as e:      # a tree that cannot be printed must not stop a job
                    logger.warning(f"could not print the experiment tree: {e}", at=None)

        return [print_exp]

    def build_before_train_hooks(self) -> list:
        """Run right after the ``after_init`` hooks, before models, optimizer and data are built."""
        return []

    def build_before_step_hooks(self) -> list:
        return []

    def build_after_step_hooks(self) -> list:
        return []

    def build_after_train_hooks(self) -> list:
        return []

    def make_logs(self, iteration: int, metrics: dict, tb_writer: Any = None) -> dict:
        """Route reduced metrics: scalars to the writer and to the console line."""
        scalars = {}
        for k, v in metrics.items():
            if torch.is_tensor(v) and v.numel() == 1:
                scalars[k] = float(v)
            elif isinstance(v, (int, float)):
                scalars[k] = v
        if tb_writer is not None:
            for k, v in scalars.items():
                tb_writer.add_scalar(k, v, iteration)
            for k, v in metrics.items():
                if torch.is_tensor(v) and v.numel() > 1:
                    tb_writer.add_histogram(str(k), v.detach().float().flatten().cpu(), iteration)
                elif isinstance(v, list) and v and isinstance(v[0], str):
                    tb_writer.add_text(str(k), "\n\n".join(v), iteration)
        return scalars

    def is_data_source(self) -> bool:
        """Ranks that read the data loader: (first or last pipeline stage), TP rank 0, CP rank 0."""
        from ..parallel.state import PM

        ends = PM.is_pipeline_first_stage(ignore_virtual=True) or PM.is_pipeline_last_stage(ignore_virtual=True)
        return ends and PM.rank_in("TP") == 0 and PM.rank_in("CP") == 0

    def sync_get_data(self, data_iterator, preprocess=None) -> dict:
        """Fetch one micro-batch where the data lives and broadcast it to the ranks that need it.

        Only (first or last pipeline stage) ∧ TP rank 0 ∧ CP rank 0 read the loader; the batch is
        broadcast over CP, then TP; ``global_data_keys`` travel over PP too (reference
        ``base_exp.py:146-221``)."""
        from ..parallel.state import PM
        from ..utils.dist_utils import broadcast_tensors

        ends = PM.is_pipeline_first_stage(ignore_virtual=True) or PM.is_pipeline_last_stage(ignore_virtual=True)
        is_src = ends and PM.rank_in("TP") == 0 and PM.rank_in("CP") == 0
        data = next(data_iterator) if is_src and data_iterator is not None else None
        dev = "cuda" if torch.cuda.is_available() else "cpu"
        if ends:
            for fam in ("CP", "TP"):
                if PM.size_of(fam) > 1:
                    data = broadcast_tensors(data, src=PM.ranks_of(fam)[0], group=PM.group_of(fam), device=dev)
        keys = self.global_data_keys
        if keys and PM.size_of("PP") > 1:
            sub = {k: data[k] for k in keys} if (data is not None and PM.is_pipeline_first_stage(True)) else None
            sub = broadcast_tensors(sub, src=PM.ranks_of("PP")[0], group=PM.group_of("PP"), device=dev)
            if data is None:
                data = dict(sub)
        if data is not None:
            from ..utils.general import recur_to

            data = recur_to(data, dev)
            if preprocess is not None:
                data = preprocess(data)
        return data


class ProfilerConfig(Config):
    timing_log_level = 0
    timing_use_event = True
    log_path = Ref("..log_path", "./")
    nvtx_ranges: bool = False
    """bracket every timed region (at the active timing level) with an NVTX range of the same name"""
    kernel_watchdog_s: float | None = None
    """seconds between reads of the kernels' status word by a watchdog thread (None: the word is read when the
    trainer logs); an error code ends training at once instead of at the next log line"""
    stall_watchdog_s: float | None = None
    """report (with the stacks of all threads) when no training step finished for this many seconds"""


class TokenizerConfig(AbstractTokenizerConfig):
    vocab_size: int = 65536
    make_vocab_size_divisible_by: int = 128
    tokenizer_path: str | None = None
    tensor_model_parallel_size: int = Ref("..model_cfg.parallel_cfg.tensor_model_parallel_size", 1)

    @writable_property
    def padded_vocab_size(self) -> int:
        from ..utils.general import make_divisible

        return make_divisible(self.vocab_size, self.make_vocab_size_divisible_by * self.tensor_model_parallel_size)

    def build_tokenizer(self):
        if self.tokenizer_path is None:
            return None
        from ..tokenizer import HFCompatTokenizer

        return HFCompatTokenizer.from_pretrained(self.tokenizer_path)


class ParallelConfig(Config):
    """Rank layout of every process-group family (reference ``base_exp.py:308-358``)."""

    parallel_definition: dict = {
        "TP": "(p d t) -> (p d) t",
        "PP": "(p d t) -> (d t) p",
        "DP": "(p d t) -> (p t) d",
        "CP": "(p d c t) -> (p d t) c",
        "MP": "(p d t) -> d (p t)",
        "EP": "(p edp ep etp) -> (p edp etp) ep",
        "ETP": "(p edp ep etp) -> (p edp ep) etp",
        "EETP": "(p edp ep etp) -> (p edp) (ep etp)",
        "EDP": "(p edp ep etp) -> (p ep etp) edp",
        "EMP": "(p edp ep etp) -> edp (p ep etp)",
    }
    tensor_model_parallel_size: int = 1
    pipeline_model_parallel_size: int = 1
    expert_model_parallel_size: int = 1
    context_parallel_size: int = 1
    expert_tensor_parallel_size: int = Ref(".tensor_model_parallel_size")
    virtual_pipeline_model_parallel_size: int = 1  # not a process-group family

    def build_parallel(self) -> dict:
        from ..parallel.state import PM

        sizes = {
            "p": self.pipeline_model_parallel_size,
            "c": self.context_parallel_size,
            "ep": self.expert_model_parallel_size,
            "t": self.tensor_model_parallel_size,
            "etp": self.expert_tensor_parallel_size,
        }
        out = {}
        for name, pattern in self.parallel_definition.items():
            axes = set(pattern.split("->")[0].replace("(", " ").replace(")", " ").split())
            out[name] = PM.define_parallel(pattern, **{k: v for k, v in sizes.items() if k in axes})
        return out

    def sanity_check(self):
        super().sanity_check()
        if os.getenv("WORLD_SIZE") is None:
            return  # not inside a launched job: the experiment checks the layout against its resource request
        world = int(os.environ["WORLD_SIZE"])
        attn = self.pipeline_model_parallel_size * self.tensor_model_parallel_size * self.context_parallel_size
        moe = self.pipeline_model_parallel_size * self.expert_tensor_parallel_size * self.expert_model_parallel_size
        assert world >= attn and world % attn == 0, f"world {world} vs PP*TP*CP {attn}"
        assert world >= moe and world % moe == 0, f"world {world} vs PP*ETP*EP {moe}"


class MegatronTPConfig(AbstractModelConfig):
    params_dtype = Ref("..params_dtype", torch.bfloat16)
    sequence_parallel: bool = False
    gradient_accumulation_fusion: bool = True
    """Weight gradients are accumulated into the fp32 ``main_grad`` by the wgrad GEMM epilogue."""
    async_tensor_model_parallel_allreduce: bool = True
    distribute_saved_activations: bool = False

    def get_tp_kwargs(self) -> dict:
        return {"params_dtype": self.params_dtype, "sequence_parallel": self.sequence_parallel}


class MegatronPPModelConfig(AbstractModelConfig):
    params_dtype: torch.dtype = torch.bfloat16
    overlap_p2p_comm: bool = True
    """Pipeline sends that are not paired with a receive (warm-up forwards, cool-down gradients) are left in flight
    on NCCL's stream instead of being waited for, so the next micro-batch's compute starts at once; exchanges that
    receive stay one batched send+receive per step and are waited for (``parallel/pipeline/p2p.py``)."""
    variable_seq_lengths: bool = False
    pp_comm_shape: tuple | None = None
    check_nan: bool = False
    """When True every stage output is checked for NaN/Inf: on the GPU by a kernel that sets a device flag (no host
    synchronisation; the trainer reads the flag when it logs and raises), on the CPU at once.  The reference
    checks on the host after every forward (``core/pipeline_parallel/schedules.py:204-205``)."""
    pipeline_activation_cpu_offload: bool = False
    fp32_residual_connection: bool = False
    fp32_output: bool = True

    def get_pp_scheduler(self):
        from ..parallel.pipeline.schedules import FWBWScheduler, PPScheduler, VPPScheduler
        from ..parallel.state import PM

        if PM.size_of("PP") > 1:
            return VPPScheduler(config=self) if PM.get_vpp_size() > 1 else PPScheduler(config=self)
        return FWBWScheduler(config=self)

    def sanity_check(self):
        super().sanity_check()
        if not self.variable_seq_lengths:
            assert self.pp_comm_shape is not None


class Megatron3DParallelModelConfig(MegatronPPModelConfig):
    tp_cfg: MegatronTPConfig = MegatronTPConfig
    parallel_cfg = ParallelConfig
    global_seq_length = Ref("..trainer_cfg.global_seq_length", 8192)
    micro_batch_size = Ref("..trainer_cfg.micro_batch_size", 1)
    hidden_size: int

    @writable_property
    def pp_comm_shape(self):
        seq = self.global_seq_length // self.parallel_cfg.context_parallel_size
        if self.tp_cfg.sequence_parallel:
            seq //= self.parallel_cfg.tensor_model_parallel_size
        return (seq * self.micro_batch_size, self.hidden_size)


class DataConfig(AbstractDataConfig):
    global_data_keys: list | None = None

    def preprocess(self, batch: dict) -> dict:
        from ..utils.general import recur_to

        return recur_to(batch, "cuda" if torch.cuda.is_available() else "cpu")


class BaseExp(Config):
    resource_cfg: ResourceConfig = ResourceConfig
    seed = 1234
    log_dir = "./"
    suffix: str = ""
    project_name = None

    @cached_property
    def file_path(self):
        return inspect.getabsfile(self.__class__)

    @writable_property
    def exp_name(self):
        base = os.path.basename(self.file_path).split(".")[0]
        return f"{base}/{self.suffix}".rstrip("/")

    @property
    def log_path(self):
        return os.path.join(self.log_dir, self.exp_name)

    @writable_property
    def exp_log_dir(self):
        """Where this experiment's logs go: ``log_dir/exp_name`` unless assigned (reference: exp/abstract.py:154-159)."""
        return os.path.join(self.log_dir, self.exp_name)

    def update_from_args(self, argv=None):
        from ..utils.logger import logger, setup_logger

        diff = self.merge(parse_args(argv), exists_only=True)
        try:
            setup_logger(self.log_path)
        except Exception:
            pass
        if diff:
            logger.info("Modified by Args:\n" + "\n".join(f"{k}: {s} -> {t}" for k, s, t in diff))
        return diff

    def build_log_writer(self):
        from ..utils.logger import StepWriter

        return StepWriter(log_dir=self.log_path, project_name=self.project_name, exp_name=self.exp_name,
                          backend=list(getattr(self.trainer_cfg, "writer_backend", ["tensorboard"])), exp=self)

    def sanity_check(self):
        """Validate the tree. When no launcher has set ``WORLD_SIZE`` the expected world size of the
        resource config is assumed for the duration of the check (and removed again afterwards, so a
        plain single-process run does not try to rendezvous with ranks that do not exist)."""
        expected = self.resource_cfg.replica * max(self.resource_cfg.gpu, 1)
        had = "WORLD_SIZE" in os.environ
        if not had:
            os.environ["WORLD_SIZE"] = str(expected)
        try:
            super().sanity_check()
        finally:
            if not had:
                del os.environ["WORLD_SIZE"]
