"""Gradient managers: gradient accumulation into fp32 flat buffers, data-parallel reduction,
global-norm clipping, the optimizer step on fp32 masters and the bf16 parameter refresh.

Reference: ``steptronoss/optimizer/base_gradient_manager.py:37-257``,
``gradient_manager.py:19-197`` (all-reduce, full optimizer state on every rank) and
``zero1_gradient_manager.py:22-243`` (reduce-scatter, optimizer state sharded over DP by whole
parameters, bf16 parameter all-gather).

What is different here:

* weight gradients arrive in ``main_grad`` from the wgrad GEMM epilogues (no per-parameter
  ``main_grad += grad`` launches); parameters whose gradient comes through autograd (CPU path,
  exotic modules) are folded in by a post-accumulate hook;
* the 1/N averaging, the clip coefficient and the bf16 cast are folded into the Adam kernel; the
  squared-norm reduction and the clip coefficient stay on the device (no ``.item()``);
* parameters are views of the flat bf16 buffer, so the parameter all-gather writes in place; it is
  issued on a side stream and joined before the next forward.
"""
from __future__ import annotations

import math

import torch
import torch.distributed as dist

from ..ops import native
from ..ops.gemm import count_launch
from ..parallel.layers import set_defaults_if_not_set_tensor_model_parallel_attributes
from ..parallel import comm
from ..parallel.state import PM
from .adam import FlatAdamShard
from .buffers import Bucket, build_buffers


class DummyOptimizer:
    """Stand-in for pipeline stages that own no trainable parameter."""

    param_groups: list = []
    optimizer = None

    def zero_grad(self, *a, **k):
        pass

    def step(self, *a, **k):
        return True, 0.0, 0

    def state_dict(self):
        return {}

    def load_state_dict(self, sd):
        pass

    def wait_param_gather(self):
        pass


def _default_wd_mult(name: str, p, on_1d: bool) -> float:
    if name.endswith(".bias") or (p.dim() == 1 and not on_1d):
        return 0.0
    return 1.0


class _ParamGroupView(dict):
    """Entry of ``optimizer.param_groups``: the scheduler writes ``lr`` / ``weight_decay`` here."""


class BaseGradientManager:
    shard_optimizer = False

    def __init__(self, cfg, model):
        self.cfg = cfg
        self.models = list(model) if isinstance(model, (list, tuple)) else [model]
        self.opt_cfg = cfg.optimizer_cfg
        self.clip_grad = float(cfg.clip_grad or 0.0)
        named = []
        for mi, m in enumerate(self.models):
            for n, p in m.named_parameters():
                set_defaults_if_not_set_tensor_model_parallel_attributes(p)
                named.append((f"model{mi}.{n}" if len(self.models) > 1 else n, p))
        seen, uniq = set(), []
        for n, p in named:
            if id(p) not in seen:
                seen.add(id(p))
                uniq.append((n, p))
        self.named_params = uniq
        if hasattr(self.opt_cfg, "mark_muon_params"):
            for m in self.models:
                self.opt_cfg.mark_muon_params(m)
        self._peer: dict = {}          # reduce group name -> PeerZeroGroup (ZeRO-1 over peer memory)
        self._peer_sq_store: dict = {}
        self.buckets: dict = build_buffers(self.named_params, shard=self.shard_optimizer,
                                           allocator=self._buffer_allocator())
        for pz in self._peer.values():
            pz.finish_allocation()
        self.step_count = 0
        self._steps_since_load = 0
        self._hooks = []
        self._install_hooks()
        self._build_optimizers()
        dev = self.named_params[0][1].device
        self.device = dev
        self.scalars = torch.zeros(4, dtype=torch.float32, device=dev)
        self.scalars[2] = 1.0
        self.scalars[3] = 1.0
        # steps whose update was applied: scalars[3] of every step added up on the device, so that the steps which a
        # non-finite gradient norm skipped can be counted at log time without a host read per step
        self.applied_steps = torch.zeros(1, dtype=torch.float32, device=dev)
        self._gather_event = None
        self._side_stream = torch.cuda.Stream() if dev.type == "cuda" else None
        self._sq_partial = None
        self._peer_sq = None
        self.optimizer = self  # `.optimizer.param_groups` is what schedulers and checkpoints use

    # ------------------------------------------------------------------ setup
    def _buffer_allocator(self):
        return None

    def _peer_of(self, key):
        pz = self._peer.get(key.reduce_group)
        return pz if pz is not None and key in pz.grad_mem else None

    def _drop_peer_path(self) -> None:
        """Move the flat buffers back to ordinary allocations (collective); the NCCL statement takes over."""
        if not self._peer:
            return
        self.wait_param_gather()
        for key, b in self.buckets.items():
            if self._peer_of(key) is None:
                continue
            if b.grad_buf is not None:
                g = b.grad_buf.clone()
                b.grad_buf = g
                for s in b.slots:
                    s.param.main_grad = g[s.offset: s.offset + s.numel].view(s.param.shape)
            if b.param_buf.is_cuda:
                self._reseat(b, b.param_buf.clone())
        for shard in self.shards.values():
            shard.peer = None
        for pz in self._peer.values():
            pz.release()
        self._peer = {}

    def _install_hooks(self) -> None:
        def hook(p):
            if p.grad is not None:
                p.main_grad.add_(p.grad.to(p.main_grad.dtype).view_as(p.main_grad))
                p.grad = None

        for _, p in self.named_params:
            if p.requires_grad:
                self._hooks.append(p.register_post_accumulate_grad_hook(hook))

    def _build_optimizers(self) -> None:
        oc = self.opt_cfg
        on_1d = bool(getattr(oc, "weight_decay_on_1d_params", False))
        self.param_groups = [_ParamGroupView(lr=float(oc.lr), weight_decay=float(oc.weight_decay), name="default")]
        self.shards: dict = {}
        self.muon = None
        muon_items = []
        for key, b in self.buckets.items():
            lo, hi = b.own_range()
            own = b.own_slots()
            if key.is_muon:
                muon_items.append((b, own))
                continue
            segs = []
            for s in own:
                lr_mult = float(oc.scale_lr_func(s.name, s.param)) if hasattr(oc, "scale_lr_func") else 1.0
                wd_mult = (float(oc.scale_wd_cond(s.name, s.param)) if hasattr(oc, "scale_wd_cond")
                           else _default_wd_mult(s.name, s.param, on_1d))
                segs.append((s.offset - lo, s.numel, lr_mult, wd_mult))
            mode = "adamw" if getattr(oc, "is_muon", False) else "adam"
            self.shards[key] = FlatAdamShard(b, lo, hi, segs, mode)
        if muon_items:
            from .muon import FlatMuon

            self.muon = FlatMuon(oc, muon_items)

    # ------------------------------------------------------------------ step pieces
    def zero_grad(self, set_to_none: bool = True) -> None:
        for pz in self._peer.values():
            pz.wait_params()   # the peers may still be reading last step's gradients
        for b in self.buckets.values():
            b.grad_buf.zero_()
        for _, p in self.named_params:
            p.grad = None
            p.grad_added_to_main_grad = False

    def wait_param_gather(self) -> None:
        """Join the side-stream parameter all-gather before parameters are read again."""
        for pz in self._peer.values():
            pz.wait_params()
        if self._gather_event is not None:
            torch.cuda.current_stream().wait_event(self._gather_event)
            self._gather_event = None

    def _allreduce_tagged(self, tag: str, group_name: str = "TP") -> None:
        """Sum the gradients of the parameters that carry ``tag`` over ``group_name`` (norm weights under sequence
        parallelism: every TP rank saw its own rows).  A bucket all of whose parameters carry the tag is reduced in
        place as one flat buffer (the usual case: the bucket of TP-replicated parameters); what is left goes through
        one packed buffer and one multi-tensor copy back."""
        if PM.size_of(group_name) == 1:
            return
        group = PM.group_of(group_name)
        rest = []
        for b in self.buckets.values():
            tagged = [s.param for s in b.slots if getattr(s.param, tag, False) and s.param.requires_grad]
            if not tagged:
                continue
            if len(tagged) == len(b.slots) and b.grad_buf is not None:
                dist.all_reduce(b.grad_buf, group=group)
            else:
                rest += [p.main_grad for p in tagged]
        in_buckets = {id(s.param) for b in self.buckets.values() for s in b.slots}
        rest += [p.main_grad for _, p in self.named_params
                 if getattr(p, tag, False) and p.requires_grad and id(p) not in in_buckets]
        if not rest:
            return
        flat = torch.cat([g.reshape(-1) for g in rest])
        dist.all_reduce(flat, group=group)
        torch._foreach_copy_(rest, [v.view_as(g) for v, g in zip(flat.split([g.numel() for g in rest]), rest)])

    def _scale_expert_grads(self) -> None:
        """Expert parameters see tokens of the whole EP group: the reference rescales their gradients
        by TP/EP so that the later 1/EDP averaging equals the data-parallel mean
        (``base_gradient_manager.py:180-200``)."""
        ep, tp = PM.size_of("EP"), PM.size_of("TP")
        if ep == 1:
            return
        factor = tp / ep
        for key, b in self.buckets.items():
            if key.reduce_group == "EDP" and factor != 1.0:
                b.grad_buf.mul_(factor)

    def _reduce(self) -> None:
        raise NotImplementedError

    def _norm_region(self, b: Bucket) -> torch.Tensor:
        raise NotImplementedError

    def _norm_group(self):
        raise NotImplementedError

    def _sqnorm_into(self, x: torch.Tensor, out: torch.Tensor, accumulate: bool) -> None:
        if x.is_cuda:
            lib = native.load()
            if self._sq_partial is None:
                self._sq_partial = torch.empty(lib.stb_sqnorm_grid(), dtype=torch.float32, device=x.device)
            native.check(lib.stb_sqnorm(x.data_ptr(), x.numel(), self._sq_partial.data_ptr(), out.data_ptr(),
                                        int(accumulate), native.stream()), "sqnorm")
            count_launch(2)
        else:
            v = x.double().pow(2).sum().float()
            out[0] = out[0] + v if accumulate else v

    def _compute_clip(self, grad_scale: float) -> None:
        """scalars[0] = global squared norm of the averaged gradient, [1] norm, [2] clip coefficient."""
        tp_rank = PM.rank_in("TP")
        regions = [self._norm_region(b) for key, b in self.buckets.items() if not (key.tp_replicated and tp_rank != 0)]
        grp = self._norm_group()
        multi = grp is not False and dist.is_initialized() and PM.world_size > 1
        if self.device.type != "cuda":
            # host path: accumulate in fp64 so that the result does not depend on how the
            # parameters are sharded over ranks
            tot = torch.zeros(1, dtype=torch.float64)
            for r in regions:
                tot += r.double().pow(2).sum()
            tot *= grad_scale * grad_scale
            if multi:
                dist.all_reduce(tot, group=grp)
            nrm = float(tot.sqrt())
            ok = math.isfinite(nrm)
            self.scalars[0] = float(tot)
            self.scalars[1] = nrm
            self.scalars[2] = (min(1.0, self.clip_grad / (nrm + 1e-6)) if self.clip_grad > 0 else 1.0) if ok else 0.0
            self.scalars[3] = 1.0 if ok else 0.0
            return
        total = self.scalars[0:1]
        if getattr(self, "_peer_sq", None) is not None:
            # the peer reduce kernels left every shard's squared norm behind: add them up instead of re-reading
            keys = [key for key in self.buckets if not (key.tp_replicated and tp_rank != 0)]
            first = True
            for key in keys:
                if key in self._peer_sq:
                    if first:
                        total.copy_(self._peer_sq[key])
                    else:
                        total.add_(self._peer_sq[key])
                else:
                    self._sqnorm_into(self._norm_region(self.buckets[key]), total, accumulate=not first)
                first = False
            regions = keys
        else:
            for i, r in enumerate(regions):
                self._sqnorm_into(r, total, accumulate=i > 0)
        if not regions:
            total.zero_()
        total.mul_(grad_scale * grad_scale)
        if multi:
            dist.all_reduce(total, group=grp)
        native.check(native.load().stb_clip_coef(self.scalars.data_ptr(), self.clip_grad, native.stream()), "clip_coef")
        count_launch()

    def _refresh_params(self) -> None:
        pass

    def _publish_loaded_shards(self) -> None:
        """After optimizer state was loaded into the owned shards: make every replica see them (no-op here)."""

    def count_zeros(self) -> torch.Tensor:
        z = torch.zeros(1, dtype=torch.float32, device=self.device)
        for b in self.buckets.values():
            r = self._norm_region(b)
            z += (r.numel() - torch.count_nonzero(r)).float()
        return z

    def _record_detailed_grad_norms(self, grad_scale: float) -> None:
        """Squared norm of the reduced gradient per ``_log_name`` (set by the model's ``name_parameters``), each
        element counted by exactly one rank: the owner under ZeRO-1, the first rank of the reduce group otherwise,
        TP rank 0 for parameters that are equal on all TP ranks.  A debugging aid: it reads every gradient once more."""
        from ..utils.metrics import GlobalMetrics

        if "grad_norms" not in GlobalMetrics.metrics:
            return
        GlobalMetrics.grad_norms.armed = True
        tp_rank = PM.rank_in("TP")
        sums: dict = {}
        for key, b in self.buckets.items():
            if key.tp_replicated and tp_rank != 0:
                continue
            if self.shard_optimizer:
                slots = b.own_slots()
            else:
                slots = b.slots if PM.rank_in(key.reduce_group) == 0 else []
            for s in slots:
                name = getattr(s.param, "_log_name", None)
                if name is None:
                    continue
                sq = b.grad_buf[s.offset:s.offset + s.numel].double().pow(2).sum() * (grad_scale * grad_scale)
                sums[name] = sums[name] + sq if name in sums else sq
        for name, sq in sums.items():
            GlobalMetrics.grad_norms.add(sq, subname=name)

    # ------------------------------------------------------------------ the step
    @torch.no_grad()
    def step(self):
        """Reduce, clip, update, refresh. Returns ``(ok, grad_norm tensor, num_zeros tensor|None)``;
        both tensors stay on the device, reading them is the caller's (logging) decision."""
        self.step_count += 1
        self._steps_since_load += 1
        self._allreduce_tagged("sequence_parallel", "TP")
        self._allreduce_tagged("micro_dp", "TP")
        self._allreduce_tagged("tp_partial_grad", "TP")
        self._scale_expert_grads()
        grad_scale = self._reduce()
        self._compute_clip(grad_scale)
        self.applied_steps.add_(self.scalars[3:4])
        zeros = self.count_zeros() if self.cfg.log_num_zeros_in_grad else None
        if getattr(self.cfg, "log_detailed_grad_norms", False):
            self._record_detailed_grad_norms(grad_scale)
        pg = self.param_groups[0]
        oc = self.opt_cfg
        for key, shard in self.shards.items():
            shard.step(self.step_count, float(pg["lr"]), float(pg["weight_decay"]), float(oc.adam_beta1),
                       float(oc.adam_beta2), float(oc.adam_eps), grad_scale, self.scalars)
        if self.muon is not None:
            self.muon.step(float(pg["lr"]), float(pg["weight_decay"]), grad_scale, self.scalars)
        self._refresh_params()
        return True, self.scalars[1], zeros

    def skipped_steps(self) -> int:
        """Steps since construction (or the last load) whose update was skipped because the gradient norm was not
        finite.  Reads one float from the device: call it where the host waits anyway (the log line).  The reference
        counts the same thing on the host per step (core/trainers/lm_trainer.py:242-298, ``N-skipped``)."""
        return self._steps_since_load - int(round(float(self.applied_steps.item())))

    # ------------------------------------------------------------------ state
    def state_dict(self) -> dict:
        sd = {"step": self.step_count, "param_groups": [dict(g) for g in self.param_groups], "buckets": {}}
        for key, shard in self.shards.items():
            sd["buckets"][str(key)] = {k: v.detach().cpu() for k, v in shard.state_dict().items()}
        if self.muon is not None:
            sd["muon"] = self.muon.state_dict()
        sd["layout"] = {str(k): [(s.name, s.owner, s.offset, s.numel) for s in b.slots] for k, b in self.buckets.items()}
        return {"optimizer": sd}

    def load_state_dict(self, state: dict) -> None:
        sd = state.get("optimizer", state)
        self.step_count = int(sd.get("step", 0))
        for g, saved in zip(self.param_groups, sd.get("param_groups", [])):
            g.update(saved)
        for key, shard in self.shards.items():
            if str(key) in sd.get("buckets", {}):
                shard.load_state_dict({k: v.to(self.device) for k, v in sd["buckets"][str(key)].items()})
                lo, hi = shard.lo, shard.hi
                shard.bucket.param_buf[lo:hi].copy_(shard.master)
        if self.muon is not None and "muon" in sd:
            self.muon.load_state_dict(sd["muon"])
        self._publish_loaded_shards()
        self._refresh_params()
        self.wait_param_gather()

    def load_resharded_state(self, read_shard, old_dp: int, strict: bool = True) -> None:
        """Restore optimizer state written by a job with ANOTHER data-parallel size.

        ``read_shard(r)`` returns what old DP rank ``r`` saved (``state_dict()`` of its manager).  Every saved shard
        lists which parameters it holds and where (``layout``); the state of each parameter this rank owns now is
        cut out of the old owner's shard by name.  Old files are read one at a time.  ``strict``: a parameter that
        the checkpoint lacks is an error; otherwise it starts from its current weights with zero moments."""
        if any(k.reduce_group == "EDP" for k in self.buckets) and PM.size_of("EP") > 1:
            raise NotImplementedError("optimizer state of expert-parallel buckets cannot be resharded; "
                                      "load the weights only (load_option.none(but=['model']))")
        first = read_shard(0)
        first = first.get("optimizer", first)
        self.step_count = int(first.get("step", 0))
        for g, saved in zip(self.param_groups, first.get("param_groups", [])):
            g.update(saved)
        self.refresh_masters_from_params()                       # the starting point of whatever is not found
        wanted: dict = {}                                        # old owner -> [(bucket key, my slot, old offset)]
        missing = []
        for key, shard in self.shards.items():
            old = {name: (owner, off, n) for name, owner, off, n in first.get("layout", {}).get(str(key), [])}
            for s in shard.bucket.own_slots():
                if s.name in old and old[s.name][2] == s.numel:
                    wanted.setdefault(old[s.name][0], []).append((key, s, old[s.name][1]))
                else:
                    missing.append(s.name)
        muon_mine = {e["slot"].name for e in self.muon.entries} if self.muon is not None else set()
        muon_found: dict = {}
        for r in range(old_dp):
            sd = first if r == 0 else read_shard(r)
            sd = sd.get("optimizer", sd)
            for key, s, old_off in wanted.get(r, []):
                saved = sd["buckets"][str(key)]
                base = r * saved["master"].numel()               # the old shard covered [base, base + shard size)
                shard = self.shards[key]
                for name in ("master", "exp_avg", "exp_avg_sq"):
                    getattr(shard, name)[s.offset - shard.lo:s.offset - shard.lo + s.numel].copy_(
                        saved[name][old_off - base:old_off - base + s.numel])
            for name, st in sd.get("muon", {}).items():
                if name in muon_mine:
                    muon_found[name] = st
        if self.muon is not None:
            self.muon.load_state_dict(muon_found)
            missing += sorted(muon_mine - set(muon_found))
        if missing and strict:
            raise RuntimeError(f"optimizer state of {len(missing)} parameters is not in the checkpoint: {missing[:5]} ...")
        for shard in self.shards.values():
            shard.bucket.param_buf[shard.lo:shard.hi].copy_(shard.master)
        self._publish_loaded_shards()
        self._refresh_params()
        self.wait_param_gather()

    def refresh_masters_from_params(self) -> None:
        """After loading model weights without optimizer state: fp32 masters follow the parameters."""
        for shard in self.shards.values():
            shard.master.copy_(shard.bucket.param_buf[shard.lo:shard.hi])
        if self.muon is not None:
            for e in self.muon.entries:
                e["master"].copy_(e["low"])

    def reload_model_params(self) -> None:
        """The reference's name for ``refresh_masters_from_params`` (optimizer/gradient_manager.py:84-87)."""
        self.refresh_masters_from_params()

    def to_device(self, device, non_blocking: bool = False) -> None:
        """Move the optimizer state (masters, moments) to ``device``: the host while another role owns the GPU, back
        before the next step.  ``non_blocking`` is accepted for call compatibility; the copies are ordered on the
        current stream either way.  Reference: optimizer/gradient_manager.py:127-151."""
        if torch.device(device).type == "cpu":
            self.offload_state()
        else:
            self.reload_state()

    # ------------------------------------------------------------------ offload (RL role swapping)
    def offload_state(self) -> None:
        for shard in self.shards.values():
            for name in ("master", "exp_avg", "exp_avg_sq"):
                setattr(shard, name, getattr(shard, name).to("cpu"))
        if self.muon is not None:
            self.muon.to("cpu")

    def reload_state(self) -> None:
        for shard in self.shards.values():
            for name in ("master", "exp_avg", "exp_avg_sq"):
                setattr(shard, name, getattr(shard, name).to(self.device))
        if self.muon is not None:
            self.muon.to(self.device)


    def destroy_buffer(self) -> None:
        """Free the fp32 gradient buffers (their contents are lost); ``build_buffer`` brings them back."""
        self._drop_peer_path()
        for b in self.buckets.values():
            b.grad_buf = None
            for s in b.slots:
                s.param.main_grad = None

    def build_buffer(self) -> None:
        for b in self.buckets.values():
            if b.grad_buf is not None:
                continue
            b.grad_buf = torch.zeros(b.numel, dtype=torch.float32, device=self.device)
            for s in b.slots:
                s.param.main_grad = b.grad_buf[s.offset : s.offset + s.numel].view(s.param.shape)
                s.param.grad_added_to_main_grad = False

    def offload_params(self, non_blocking: bool = True) -> None:
        """Move the flat parameter buffers to pinned host memory; parameters stay views of them."""
        self._drop_peer_path()
        self.wait_param_gather()
        for b in self.buckets.values():
            if b.param_buf.device.type == "cpu":
                continue
            host = torch.empty(b.param_buf.shape, dtype=b.param_buf.dtype, device="cpu",
                               pin_memory=torch.cuda.is_available())
            host.copy_(b.param_buf, non_blocking=non_blocking)
            self._reseat(b, host)
        if torch.cuda.is_available():
            torch.cuda.current_stream().synchronize()

    def reload_params(self, non_blocking: bool = True) -> None:
        for b in self.buckets.values():
            if b.param_buf.device == self.device:
                continue
            dev = torch.empty(b.param_buf.shape, dtype=b.param_buf.dtype, device=self.device)
            dev.copy_(b.param_buf, non_blocking=non_blocking)
            self._reseat(b, dev)

    @staticmethod
    def _reseat(b: Bucket, buf: torch.Tensor) -> None:
        b.param_buf = buf
        for s in b.slots:
            s.param.data = buf[s.offset : s.offset + s.numel].view(s.param.shape)


GradientManager = BaseGradientManager      # the reference's name for the base (optimizer/base_gradient_manager.py)


class AccInFP32GradientManager(BaseGradientManager):
    """All-reduce gradients over DP; every rank keeps the full optimizer state."""

    shard_optimizer = False

    def _reduce(self) -> float:
        scale = 1.0
        for key, b in self.buckets.items():
            n = PM.size_of(key.reduce_group)
            if n > 1:
                dist.all_reduce(b.grad_buf, group=PM.group_of(key.reduce_group))
            scale = 1.0 / PM.size_of("DP")
        self._edp_fix(scale)
        return scale

    def _edp_fix(self, scale: float) -> None:
        # buckets reduced over EDP are averaged over a smaller group than DP
        dp, edp = PM.size_of("DP"), PM.size_of("EDP") if PM.has("EDP") else PM.size_of("DP")
        if edp != dp:
            for key, b in self.buckets.items():
                if key.reduce_group == "EDP":
                    b.grad_buf.mul_(dp / edp)

    def _norm_region(self, b):
        return b.grad_buf

    def _norm_group(self):
        return PM.group_of("MP") if PM.has("MP") and PM.size_of("MP") > 1 else False


class Zero1GradientManager(BaseGradientManager):
    """Reduce-scatter gradients over DP (EDP for experts); optimizer state only for owned parameters;
    bf16 parameter all-gather in place."""

    shard_optimizer = True

    def _buffer_allocator(self):
        """Buckets whose reduce group sits inside one node get their flat buffers in peer-mapped memory."""
        from . import peer_zero

        dev = self.named_params[0][1].device if self.named_params else torch.device("cpu")
        if dev.type != "cuda":
            return None
        supported: dict = {}

        def allocator(key, numel, dtype, kind):
            if key.is_muon or key.dtype != torch.bfloat16:
                return None
            g = key.reduce_group
            if g not in supported:
                supported[g] = peer_zero.group_supported(g)
                if supported[g]:
                    self._peer[g] = peer_zero.PeerZeroGroup(g)
            return self._peer[g].allocate(key, numel, dtype, kind) if supported[g] else None

        return allocator

    def _build_optimizers(self) -> None:
        super()._build_optimizers()
        for key, shard in self.shards.items():
            pz = self._peer_of(key)
            if pz is not None:
                shard.peer = (pz, pz.param_ptrs(key, self.buckets[key]))

    def _reduce(self) -> float:
        dp, edp = PM.size_of("DP"), PM.size_of("EDP") if PM.has("EDP") else PM.size_of("DP")
        for pz in self._peer.values():
            pz.begin_step()
        self._peer_sq = {} if self._peer else None
        for key, b in self.buckets.items():
            fix = dp / edp if key.reduce_group == "EDP" and edp != dp else 1.0
            pz = self._peer_of(key)
            if pz is not None:
                if key not in self._peer_sq_store:
                    self._peer_sq_store[key] = torch.zeros(1, dtype=torch.float32, device=self.device)
                self._peer_sq[key] = self._peer_sq_store[key]
                pz.reduce(key, b, fix, self._peer_sq[key], accumulate=False)
                continue
            lo, hi = b.own_range()
            if b.world > 1:
                comm.reduce_scatter_tensor(b.grad_buf[lo:hi], b.grad_buf, group=PM.group_of(key.reduce_group))
            if fix != 1.0:
                b.grad_buf[lo:hi].mul_(fix)
        return 1.0 / dp

    def _norm_region(self, b):
        lo, hi = b.own_range()
        return b.grad_buf[lo:hi]

    def _norm_group(self):
        return None  # world

    def _publish_loaded_shards(self) -> None:
        # Buckets on the peer-memory path have no all-gather in `_refresh_params` (their Adam kernel stores the new
        # shard into every rank's buffer), so shards that were just loaded from a checkpoint would stay local.
        # The buffers are this rank's own mapping: NCCL never sees a peer pointer.
        for key, b in self.buckets.items():
            if b.world > 1 and self._peer_of(key) is not None:
                lo, hi = b.own_range()
                comm.all_gather_into_tensor(b.param_buf, b.param_buf[lo:hi], group=PM.group_of(key.reduce_group))

    def _refresh_params(self) -> None:
        for pz in self._peer.values():
            pz.end_step()      # the Adam kernels already stored the new shards into every peer's buffer
        multi = [(k, b) for k, b in self.buckets.items() if b.world > 1 and self._peer_of(k) is None]
        if not multi:
            return
        if self._side_stream is not None and self.cfg.overlap_param_gather:
            self._side_stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(self._side_stream):
                for key, b in multi:
                    lo, hi = b.own_range()
                    comm.all_gather_into_tensor(b.param_buf, b.param_buf[lo:hi], group=PM.group_of(key.reduce_group))
                self._gather_event = torch.cuda.Event()
                self._gather_event.record(self._side_stream)
        else:
            for key, b in multi:
                lo, hi = b.own_range()
                comm.all_gather_into_tensor(b.param_buf, b.param_buf[lo:hi], group=PM.group_of(key.reduce_group))
