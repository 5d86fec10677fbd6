"""Mixture-of-experts block: router, grouped experts, expert-parallel dispatch, shared expert.

Reference: ``steptronoss/model/common/moe_block.py:44-491`` and ``moe_share_expert_ffn.py:13-76``.

* ``MoEGate``: router projection, optionally with fp32 output.
* ``forward_router``: softmax or sigmoid probabilities; top-k by stable descending order (ties go to
  the lower expert id); an aux-loss-free balance bias takes part in the selection only; optional
  renormalisation of the selected weights; aux loss ``E * sum(mean_prob * count)`` with the counts
  summed over the TP and EP groups.
* ``GroupedExperts``: stacked expert weights ``w1 [E/EP, 2F, H]`` (gate | up) and ``w2 [E/EP, H, F]``.
* EP path: dispatch -> experts -> combine; TP path: gather the sequence-parallel tokens, run the
  experts, keep this rank's slice.
"""
from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn as nn

from ...config import Config, Ref
from ...ops import linear
from ...ops import moe as moe_ops
from ...parallel import mappings
from ...parallel.random import checkpoint
from ...parallel.state import PM
from ...utils.metrics import GlobalMetrics
from .feed_forward import FeedForward, FeedForwardConfig


class MoEConfig(Config):
    tp_cfg = Ref("..tp_cfg")
    params_dtype = Ref("..params_dtype", torch.bfloat16)
    hidden_size: int
    moe_num_experts: int
    moe_top_k: int
    moe_aux_loss_coef: float = 0.0
    moe_hidden_size: int
    fp32_gate_output: bool = False
    routed_scaling_factor: float = 1.0
    enable_sigmoid_router: bool = False
    router_bias_update_rate: float = 0.0
    enable_auxiliary_loss_free_load_balance: bool = False
    norm_expert_weight: bool = True
    force_balance: bool = False
    moe_layer_list: list = []
    share_expert_dim: int = 0
    dispatcher: str = "alltoall"
    """``alltoall`` (NCCL all-to-all of packed rows) or ``peer`` (rows written straight into the
    destination rank's expert-major buffer over NVLink)."""
    capacity_factor: float | None = None
    """peer dispatcher only.  None: expert buffers sized by the exact number of arrived slots (one host read per
    layer).  f >= 1: sized for f x (tokens x top-k) without a host read; a rank that receives more fails the step
    with a capacity error (nothing is dropped silently)."""
    recompute_experts: bool = False
    fp8: bool = False
    """Forward products of the routed expert GEMMs in block-scaled e4m3 (1 x 128 activation scales, 128 x 128 weight
    scales, fp32 accumulation); the backward products stay in bf16."""
    detailed_router_metrics: bool = False
    """Also fill ``router_logits_std`` and ``moe_minp / moe_sumk / moe_std / moe_avg`` (per-token statistics of the
    router probabilities, as the reference logs them).  They are computed with ordinary tensor operations over the
    ``[tokens, experts]`` probabilities, about ten small launches per layer and micro-batch, so they are a
    diagnostic switch; ``router_logits_max``, ``moe_max`` and ``expert_coef`` come out of the fused router kernel
    and are always filled."""

    def get_aux_loss_calib_scale(self):
        return 1

    def get_experts_swiglu_limit(self, layer_id):
        return None

    def get_shared_expert_swiglu_limit(self, layer_id):
        return None


class _BindAuxLoss(torch.autograd.Function):
    """Identity on ``x`` that makes ``aux`` part of the graph: backward feeds gradient 1 (times the
    loss scale carried by the incoming gradient's convention) into ``aux``."""

    @staticmethod
    def forward(ctx, x, aux):
        ctx.aux_shape = aux.shape
        ctx.scale = getattr(_BindAuxLoss, "loss_scale", 1.0)
        return x

    @staticmethod
    def backward(ctx, g):
        return g, torch.full(ctx.aux_shape, ctx.scale, dtype=torch.float32, device=g.device)


AuxLossBackwardHook = _BindAuxLoss          # the reference's name (model/utils/utils.py)


def bind_aux_loss(x, aux):
    return _BindAuxLoss.apply(x, aux)


def set_aux_loss_scale(scale: float) -> None:
    """Scale applied to every auxiliary loss gradient (1 / number of micro-batches)."""
    _BindAuxLoss.loss_scale = float(scale)


class MoEGate(nn.Module):
    def __init__(self, cfg: MoEConfig):
        super().__init__()
        self.fp32 = bool(cfg.fp32_gate_output)
        self.weight = nn.Parameter(torch.empty(cfg.moe_num_experts, cfg.hidden_size, dtype=cfg.params_dtype))
        self.weight.sequence_parallel = bool(cfg.tp_cfg.sequence_parallel)

    def forward(self, x):
        if x.is_cuda and x.dtype == torch.bfloat16 and self.weight.dtype == torch.bfloat16:
            # one tcgen05 GEMM with fp32 accumulators written out as fp32: for bf16 operands this is the product that
            # ``fp32_gate_output`` asks for (the conversions to fp32 are exact), and without the flag it saves the cast
            return linear(x, self.weight, out_dtype=torch.float32)
        if self.fp32:
            return torch.nn.functional.linear(x.float(), self.weight.float())
        return linear(x, self.weight).float()


class GroupedExperts(nn.Module):
    def __init__(self, cfg: MoEConfig, layer_id: int):
        super().__init__()
        ep = PM.size_of("EP")
        if cfg.moe_num_experts % ep:
            raise ValueError(f"{cfg.moe_num_experts} experts not divisible by EP={ep}")
        self.num_local = cfg.moe_num_experts // ep
        F, H = cfg.moe_hidden_size, cfg.hidden_size
        self.w1 = nn.Parameter(torch.empty(self.num_local, 2 * F, H, dtype=cfg.params_dtype))
        self.w2 = nn.Parameter(torch.empty(self.num_local, H, F, dtype=cfg.params_dtype))
        for w in (self.w1, self.w2):
            w.expert_model_parallel = ep > 1
        lim = cfg.get_experts_swiglu_limit(layer_id)
        self.limit = float(lim) if lim else 0.0
        self.fp8 = bool(getattr(cfg, "fp8", False))

    def forward(self, x, local_ids, weights, max_slots=None):
        return moe_ops.routed_grouped_ffn(x, local_ids, weights, self.w1, self.w2, self.limit, max_slots, fp8=self.fp8)


class MoEBlock(nn.Module):
    def __init__(self, cfg: MoEConfig, layer_id: int):
        super().__init__()
        self.cfg = cfg
        self.layer_id = layer_id
        self.moe_layer_id = cfg.moe_layer_list.index(layer_id) if layer_id in cfg.moe_layer_list else layer_id
        self.num_experts, self.top_k = cfg.moe_num_experts, cfg.moe_top_k
        self.gate = MoEGate(cfg)
        self.experts = GroupedExperts(cfg, layer_id)
        self.sequence_parallel = bool(cfg.tp_cfg.sequence_parallel) and PM.size_of("TP") > 1
        if cfg.enable_auxiliary_loss_free_load_balance:
            self.register_buffer("router_balance_bias", torch.zeros(cfg.moe_num_experts, dtype=torch.float32))
            self.register_buffer("local_tokens_per_expert", torch.zeros(cfg.moe_num_experts, dtype=torch.int32),
                                 persistent=False)
        else:
            self.router_balance_bias = None
            self.local_tokens_per_expert = None
        self.micro_batch_count = 0
        self._dispatcher = None

    def maintain_float32_router_balance_bias(self) -> None:
        """The selection bias moves by ``router_bias_update_rate`` (1e-3) per step: in bf16 such steps vanish next to a
        bias of order one.  Whatever cast the module went through, the buffer is put back to fp32
        (reference: model/common/moe_block.py:423-436)."""
        b = self.router_balance_bias
        if b is not None and b.dtype != torch.float32:
            self.router_balance_bias.data = b.data.float()

    def _apply(self, fn, recurse=True):
        out = super()._apply(fn, recurse)
        self.maintain_float32_router_balance_bias()
        return out

    def _load_from_state_dict(self, *args, **kwargs):
        self.maintain_float32_router_balance_bias()
        return super()._load_from_state_dict(*args, **kwargs)

    # ------------------------------------------------------------------ router
    def forward_router(self, logits):
        cfg = self.cfg
        logits = logits.float()
        eps = 1e-20 if self.router_balance_bias is not None else 0.0
        route = (moe_ops.fused_router if moe_ops.router_native_ok(logits, self.top_k) and not cfg.force_balance
                 else moe_ops.router_reference)
        ids, weights, prob_sum, hist, stats = route(logits, self.router_balance_bias, self.top_k,
                                                    bool(cfg.enable_sigmoid_router), bool(cfg.norm_expert_weight), eps)
        if cfg.force_balance:
            base = torch.arange(logits.shape[0] * self.top_k, device=logits.device)
            ids = (base % self.num_experts).view(-1, self.top_k)
            prob = torch.sigmoid(logits) if cfg.enable_sigmoid_router else torch.softmax(logits, dim=1)
            top_prob = prob.gather(1, ids)
            weights = (top_prob / (top_prob.sum(-1, keepdim=True) + eps)
                       if cfg.enable_sigmoid_router or cfg.norm_expert_weight else top_prob)
            hist = moe_ops.histogram(ids, self.num_experts)
        ce = hist.float()
        for fam in ("TP", "EP"):
            if PM.size_of(fam) > 1:
                dist.all_reduce(ce, group=PM.group_of(fam))
        me = prob_sum / max(logits.shape[0], 1)
        if self.local_tokens_per_expert is not None and self.training:
            with torch.no_grad():
                self.local_tokens_per_expert += hist
                self.micro_batch_count += 1
        aux = (me * ce).sum() * self.num_experts
        sub = f"layer{self.moe_layer_id}"
        with torch.no_grad():
            GlobalMetrics.router_logits_max.add(stats[0], subname=sub)
            GlobalMetrics.expert_coef.add(stats[2] if stats.numel() > 2 and not cfg.force_balance
                                          else hist.max().float() / hist.sum().clamp_min(1).float(), subname=sub)
            GlobalMetrics.moe_max.add(stats[1], subname=sub)
            if cfg.detailed_router_metrics:
                lg = logits.detach().float()
                prob = torch.sigmoid(lg) if cfg.enable_sigmoid_router else torch.softmax(lg, dim=1)
                if cfg.enable_sigmoid_router:
                    prob = prob / (prob.sum(-1, keepdim=True) + eps)
                GlobalMetrics.router_logits_std.add(lg.std(1).mean(), subname=sub)
                GlobalMetrics.moe_minp.add(prob.min(1).values.mean(), subname=sub)
                GlobalMetrics.moe_sumk.add(prob.topk(self.top_k, dim=1).values.sum(1).mean(), subname=sub)
                GlobalMetrics.moe_std.add(prob.std(1).mean(), subname=sub)
                GlobalMetrics.moe_avg.add(prob.mean(1).mean(), subname=sub)
        return ids, weights, aux

    # ------------------------------------------------------------------ expert paths
    @property
    def dispatcher(self):
        if self._dispatcher is None:
            from ...parallel.ep_dispatcher import build_dispatcher

            self._dispatcher = build_dispatcher(self.cfg.dispatcher, "EP", self.num_experts,
                                                getattr(self.cfg, "capacity_factor", None))
        return self._dispatcher

    def forward_experts_tp(self, x, ids, weights):
        if self.sequence_parallel:
            x = mappings.gather_from_sequence_parallel_region(x, "TP")
            ids = mappings.gather_from_sequence_parallel_region_no_reduce(ids, "TP")
            weights = mappings.gather_from_sequence_parallel_region(weights, "TP")
        y = self.experts(x, ids, weights)
        if self.sequence_parallel:
            y = mappings.slice_sequence_parallel_region(y, "TP")
        return y

    def forward_experts_ep(self, x, ids, weights):
        n_tok = x.shape[0]
        xd, local_ids, wd = self.dispatcher.dispatch(x, ids, weights)
        with torch.no_grad():
            GlobalMetrics.peak_to_avg_ratio.add((local_ids >= 0).sum().float() / max(n_tok * self.top_k, 1),
                                                subname=f"layer{self.moe_layer_id}")
        y = self.experts(xd, local_ids, wd, getattr(self.dispatcher, "received_slots", None))
        return self.dispatcher.combine(y)

    def forward(self, x, recompute: bool = False):
        shape = x.shape
        x2 = x.reshape(-1, shape[-1])
        ids, weights, aux = self.forward_router(self.gate(x2))
        weights = weights.to(torch.float32)
        ep = PM.size_of("EP") > 1
        fn = self.forward_experts_ep if ep else self.forward_experts_tp
        if (recompute or self.cfg.recompute_experts) and torch.is_grad_enabled():
            out = checkpoint(fn, x2, ids, weights)
        else:
            out = fn(x2, ids, weights)
        if self.cfg.moe_aux_loss_coef:
            # the reference divides by TP on the expert-parallel path and by ETP (= 1) otherwise
            # (model/common/moe_block.py:394,407); kept, so that a coefficient tuned there means the same here
            aux = aux * (self.cfg.moe_aux_loss_coef / (PM.size_of("TP") if ep else max(PM.size_of("ETP"), 1)))
            out = bind_aux_loss(out, aux)
            GlobalMetrics.moe_aux_loss.add(aux.detach(), subname=f"layer{self.moe_layer_id}")
        if self.cfg.routed_scaling_factor != 1.0:
            out = out * self.cfg.routed_scaling_factor
        return out.reshape(shape)

    # ------------------------------------------------------------------ aux-loss-free balancing
    @staticmethod
    @torch.no_grad()
    def update_router_balance_bias_per_gbs(model: nn.Module) -> None:
        """Once per optimizer step: bias += rate * sign(mean_tokens - tokens) per expert, from the token
        counts summed over the ETP, EP and EDP groups; the result is averaged over DP."""
        layers = [m for m in model.modules() if isinstance(m, MoEBlock) and m.router_balance_bias is not None
                  and m.micro_batch_count > 0]
        if not layers:
            return
        tokens = torch.stack([m.local_tokens_per_expert for m in layers]).float()
        for fam in ("ETP", "EP", "EDP"):
            if PM.has(fam) and PM.size_of(fam) > 1:
                dist.all_reduce(tokens, group=PM.group_of(fam))
        new_bias = []
        for t, m in zip(tokens, layers):
            offset = t.mean(-1, keepdim=True) - t
            new_bias.append(m.router_balance_bias + torch.sign(offset) * m.cfg.router_bias_update_rate)
        stacked = torch.stack(new_bias)
        if PM.size_of("DP") > 1:
            dist.all_reduce(stacked, group=PM.group_of("DP"))
            stacked /= PM.size_of("DP")
        for m, b in zip(layers, stacked):
            m.router_balance_bias.copy_(b)
            m.local_tokens_per_expert.zero_()
            m.micro_batch_count = 0


class MoEFeedForwardConfig(FeedForwardConfig):
    moe_cfg: MoEConfig = Ref("..moe_cfg")

    def build_model(self, layer_id: int = 0):
        if layer_id in self.moe_cfg.moe_layer_list:
            return MoeShareExpertFFN(self.moe_cfg, self, layer_id)
        return FeedForward(self, layer_id)


class MoeShareExpertFFN(nn.Module):
    """Routed experts plus an optional always-on shared expert (a dense TP feed-forward)."""

    def __init__(self, moe_cfg: MoEConfig, ffn_cfg: FeedForwardConfig, layer_id: int):
        super().__init__()
        self.moe = MoEBlock(moe_cfg, layer_id)
        self.enable_share_expert = moe_cfg.share_expert_dim > 0
        if self.enable_share_expert:
            self.share_expert = FeedForward(ffn_cfg, layer_id, ffn_hidden_size=moe_cfg.share_expert_dim)
            lim = moe_cfg.get_shared_expert_swiglu_limit(layer_id)
            if lim:
                self.share_expert.limit = float(lim)

    def _log_norm(self, t, which: str) -> None:
        # mean row norm of the routed and of the shared branch (reference: model/common/moe_share_expert_ffn.py:59-74);
        # computed only where an experiment registers the metric - its default metric sets do not
        if "shared_routed_avgnorm" in GlobalMetrics:
            with torch.no_grad():
                GlobalMetrics.shared_routed_avgnorm.add(t.detach().float().norm(dim=-1).mean(),
                                                        subname=f"layer{self.moe.moe_layer_id}.{which}")

    def forward(self, x, recompute: bool = False):
        out = self.moe(x, recompute=recompute)
        self._log_norm(out, "routed")
        if self.enable_share_expert:
            shared = self.share_expert(x)
            self._log_norm(shared, "shared")
            out = out + shared
        return out
