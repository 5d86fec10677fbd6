"""Composable weight transformations between the HF layout and the native (sharded) layout.

A ``ReshapeOp`` maps a *piece* (``dict name -> tensor`` or, after a split, ``name -> list of per-rank
tensors``) forward (HF -> native) and backward (native -> HF); ops compose with ``+``.  The set of
ops follows the reference (``steptronoss/checkpointing/reshape_ops.py:34-627``): ``VocabPad``,
``ColumnParallel``, ``RowParallel``, ``Duplicate``, ``KeepThisTP``, ``KeepThisEP``, ``GQAMergeQKV``
(+bias, +gate variants), ``FFNMergeGateUp``, ``UnbindMoE``, ``MHA_TP_CHUNK``, ``Rename``, ``Inverse``,
``Sequential``, ``Script`` and ``OnlineReshaper``.

Native fused layouts of this framework: ``wqkv`` rows per TP shard are ``[q heads | k heads | v heads |
gate]`` and ``w1`` rows are ``[gate | up]``.
"""
from __future__ import annotations

import os

import contextlib
import fnmatch
import re

import torch
import torch.distributed as dist

from ..config import DataClass
from ..parallel.state import PM


def _size(group: str) -> int:
    return PM.size_of(group) if PM.has(group) else 1


def _rank(group: str) -> int:
    return PM.rank_in(group) if PM.has(group) else 0


def common_pattern(strs: list) -> str:
    """What a family of names shares: ``['aan', 'abn', 'acn'] -> 'a{}n'`` (one name comes back unchanged)."""
    names = sorted(set(strs))
    if len(names) == 1:
        return names[0]
    head = os.path.commonprefix(names)
    tail = os.path.commonprefix([n[len(head):][::-1] for n in names])[::-1]
    return f"{head}{{}}{tail}"


class ReshapeOp:
    def forward(self, piece: dict) -> dict:
        raise NotImplementedError

    def backward(self, piece: dict) -> dict:
        raise NotImplementedError

    def __add__(self, other: "ReshapeOp") -> "Sequential":
        left = self.ops if isinstance(self, Sequential) else [self]
        right = other.ops if isinstance(other, Sequential) else [other]
        return Sequential(left + right)

    def __repr__(self) -> str:
        return type(self).__name__


class Identity(ReshapeOp):
    def forward(self, piece):
        return piece

    def backward(self, piece):
        return piece


class Sequential(ReshapeOp):
    def __init__(self, ops: list):
        self.ops = list(ops)

    def forward(self, piece):
        for op in self.ops:
            piece = op.forward(piece)
        return piece

    def backward(self, piece):
        for op in reversed(self.ops):
            piece = op.backward(piece)
        return piece

    def append(self, op: ReshapeOp):
        self.ops.append(op)

    def __repr__(self):
        return " + ".join(repr(o) for o in self.ops) or "Identity"


class Inverse(ReshapeOp):
    def __init__(self, op: ReshapeOp):
        self.op = op

    def forward(self, piece):
        return self.op.backward(piece)

    def backward(self, piece):
        return self.op.forward(piece)


class Rename(ReshapeOp):
    """``"dst: src"`` (or a dict ``{dst: src}``): forward renames src -> dst, backward dst -> src.  Both sides may
    hold ``*`` wildcards (``"encoder.*: *"``, ``"a.*.fc1.*: a.*.c_fc.*"``): what the wildcards of one side capture
    fills the wildcards of the other, in order.  A piece of one tensor under a rule without wildcards takes the
    rule's name whatever it was called before (the product of a merge)."""

    def __init__(self, mapping):
        if isinstance(mapping, str):
            dst, src = (s.strip() for s in mapping.split(":"))
            mapping = {dst: src}
        self.mapping = dict(mapping)

    @staticmethod
    def _apply(piece: dict, pairs: list) -> dict:
        """``pairs``: (from, to) names or globs; the first pair that matches a key renames it."""
        from ..utils.weight_loader import fill_target, key_pattern

        globs = [(key_pattern(a), b) for a, b in pairs if "*" in a]
        exact = {a: b for a, b in pairs if "*" not in a}
        out = {}
        for k, v in piece.items():
            if k in exact:
                out[exact[k]] = v
                continue
            for pat, target in globs:
                m = pat.match(k)
                if m:
                    out[fill_target(m, target)] = v
                    break
            else:
                out[k] = v
        return out

    def forward(self, piece):
        if len(piece) == 1 and len(self.mapping) == 1:
            (dst, src), (k, v) = next(iter(self.mapping.items())), next(iter(piece.items()))
            if "*" not in dst and "*" not in src and k != src:
                return {dst: v}
        return self._apply(piece, [(src, dst) for dst, src in self.mapping.items()])

    def backward(self, piece):
        return self._apply(piece, list(self.mapping.items()))


class Prefixed(ReshapeOp):
    """A sub-module's own mapping inside a larger one: forward takes HF names below ``hf_prefix``, strips it, applies
    ``hf_names`` (pairs of HF spelling -> the spelling ``inner`` expects, as globs), runs ``inner`` and puts
    ``native_prefix`` in front; backward is the way back."""

    def __init__(self, inner: ReshapeOp, hf_prefix: str, native_prefix: str, hf_names: list | None = None,
                 mesh=None):
        self.inner, self.hf_prefix, self.native_prefix = inner, hf_prefix, native_prefix
        self.hf_names = list(hf_names or [])
        self.mesh = mesh
        """ParallelConfig of the sub-module when it lives on a mesh of its own (its TP size decides the splits)"""

    def _on_mesh(self):
        return PM.use_mesh(self.mesh) if self.mesh is not None else contextlib.nullcontext()

    def forward(self, piece):
        n = len(self.hf_prefix)
        sub = {k[n:]: v for k, v in piece.items() if k.startswith(self.hf_prefix)}
        sub = Rename._apply(sub, self.hf_names)
        with self._on_mesh():
            out = self.inner.forward(sub)
        return {self.native_prefix + k: v for k, v in out.items()}

    def backward(self, piece):
        n = len(self.native_prefix)
        sub = {k[n:]: v for k, v in piece.items() if k.startswith(self.native_prefix)}
        with self._on_mesh():
            out = self.inner.backward(sub)
        out = Rename._apply(out, [(b, a) for a, b in self.hf_names])
        return {self.hf_prefix + k: v for k, v in out.items()}


class VocabPad(ReshapeOp):
    """Pad (forward) / crop (backward) the vocabulary dimension to the model's padded size."""

    def __init__(self, target_vocab_size: int, dim: int = 0, pad_type: str = "last", actual_vocab_size: int | None = None):
        self.target, self.dim, self.pad_type, self.actual = target_vocab_size, dim, pad_type, actual_vocab_size

    def forward(self, piece):
        out = {}
        for k, t in piece.items():
            n = t.shape[self.dim]
            if self.actual is None:
                self.actual = n
            if n < self.target:
                shape = list(t.shape)
                shape[self.dim] = self.target - n
                if self.pad_type == "last":
                    fill = t.select(self.dim, n - 1).unsqueeze(self.dim).expand(shape)
                else:
                    fill = torch.zeros(shape, dtype=t.dtype, device=t.device)
                t = torch.cat([t, fill], dim=self.dim)
            elif n > self.target:
                t = t.narrow(self.dim, 0, self.target)
            out[k] = t
        return out

    def backward(self, piece):
        n = self.actual or self.target
        return {k: t.narrow(self.dim, 0, min(n, t.shape[self.dim])) for k, t in piece.items()}


class _Split(ReshapeOp):
    dim = 0

    def __init__(self, group: str = "TP"):
        self.group = group

    def forward(self, piece):
        n = _size(self.group)
        return {k: list(t.chunk(n, dim=self.dim)) for k, t in piece.items()}

    def backward(self, piece):
        return {k: torch.cat(list(parts), dim=self.dim) for k, parts in piece.items()}


class ColumnParallel(_Split):
    dim = 0


class RowParallel(_Split):
    dim = -1  # also right for stacked expert weights [E, out, in]


class Duplicate(ReshapeOp):
    def __init__(self, group: str = "TP"):
        self.group = group

    def forward(self, piece):
        n = _size(self.group)
        return {k: [t] * n for k, t in piece.items()}

    def backward(self, piece):
        return {k: parts[0] for k, parts in piece.items()}


def _all_gather_tensor(t: torch.Tensor, group: str) -> list:
    n = _size(group)
    if n == 1 or not dist.is_initialized():
        return [t]
    g = PM.group_of(group)
    dev = t.device
    if dist.get_backend(g) == "nccl" and not t.is_cuda:
        t = t.cuda()
    parts = [torch.empty_like(t) for _ in range(n)]
    dist.all_gather(parts, t.contiguous(), group=g)
    return [p.to(dev) for p in parts]


class KeepThisTP(ReshapeOp):
    """Forward keeps this rank's shard of a split piece; backward all-gathers the shards of the group."""

    def __init__(self, group: str = "TP"):
        self.group = group

    def forward(self, piece):
        r = _rank(self.group)
        return {k: parts[r].contiguous() for k, parts in piece.items()}

    def backward(self, piece):
        return {k: _all_gather_tensor(t, self.group) for k, t in piece.items()}


class KeepThisEP(ReshapeOp):
    """Stacked expert tensors ``[E, ...]``: forward keeps the experts of this EP rank, backward gathers."""

    def __init__(self, group: str = "EP", dim: int = 0):
        self.group, self.dim = group, dim

    def forward(self, piece):
        n, r = _size(self.group), _rank(self.group)
        return {k: t.chunk(n, dim=self.dim)[r].contiguous() for k, t in piece.items()}

    def backward(self, piece):
        return {k: torch.cat(_all_gather_tensor(t, self.group), dim=self.dim) for k, t in piece.items()}


class MHA_TP_CHUNK(ReshapeOp):  # noqa: N801
    """Fused ``[3, heads, d]`` multi-head projection (ViT): split so every rank gets its heads of q, k and v."""

    def __init__(self, group: str = "TP"):
        self.group = group

    def forward(self, piece):
        n = _size(self.group)
        out = {}
        for k, t in piece.items():
            three = t.chunk(3, dim=0)
            out[k] = [torch.cat([x.chunk(n, dim=0)[r] for x in three], dim=0) for r in range(n)]
        return out

    def backward(self, piece):
        out = {}
        for k, parts in piece.items():
            split = [p.chunk(3, dim=0) for p in parts]
            out[k] = torch.cat([torch.cat([s[i] for s in split], dim=0) for i in range(3)], dim=0)
        return out


class GQAMergeQKV(ReshapeOp):
    """``q_proj / k_proj / v_proj`` (+ optional gate rows) -> fused ``wqkv`` shards ``[q | k | v | gate]``."""

    suffix = "weight"

    def __init__(self, group_num: int, head_dim: int, gate_dims: int = 0, group: str = "TP"):
        self.kv_heads, self.head_dim, self.gate_dims, self.group = group_num, head_dim, gate_dims, group

    def _find(self, piece, tag):
        for k in piece:
            if f".{tag}_proj." in k or k.endswith(f"{tag}_proj.{self.suffix}") or f"{tag}_proj" in k:
                return k
        raise KeyError(f"no {tag}_proj in {list(piece)}")

    def forward(self, piece):
        n = _size(self.group)
        kq, kk, kv = (self._find(piece, t) for t in "qkv")
        blocks = [piece[kq], piece[kk], piece[kv]]
        gate_key = next((k for k in piece if "g_proj" in k or "gate_proj" in k and "mlp" not in k), None)
        if self.gate_dims and gate_key is not None:
            blocks.append(piece[gate_key])
        shards = [torch.cat([b.chunk(n, dim=0)[r] for b in blocks], dim=0) for r in range(n)]
        name = re.sub(r"[qkv]_proj", "qkv_proj", kq)
        self._names = (kq, kk, kv, gate_key if len(blocks) == 4 else None)
        return {name: shards}

    def backward(self, piece):
        (name, shards), = piece.items()
        n = len(shards)
        rows = shards[0].shape[0]
        g = self.gate_dims // n if self.gate_dims else 0
        kvr = self.kv_heads * self.head_dim // n
        qr = rows - 2 * kvr - g
        qs, ks, vs, gs = [], [], [], []
        for s in shards:
            q, k, v, gg = s.split([qr, kvr, kvr, g], dim=0)
            qs.append(q), ks.append(k), vs.append(v), gs.append(gg)
        out = {name.replace("qkv_proj", "q_proj"): torch.cat(qs), name.replace("qkv_proj", "k_proj"): torch.cat(ks),
               name.replace("qkv_proj", "v_proj"): torch.cat(vs)}
        if g:
            out[name.replace("qkv_proj", "g_proj")] = torch.cat(gs)
        return out


class GQAMergeQKVBias(GQAMergeQKV):
    suffix = "bias"


class GQAMergeQKVG(GQAMergeQKV):
    def __init__(self, group_num: int, head_dim: int, gate_dims: int, group: str = "TP"):
        super().__init__(group_num, head_dim, gate_dims, group)


class FFNMergeGateUp(ReshapeOp):
    """``gate_proj`` and ``up_proj`` -> fused ``w1`` shards ``[gate | up]``."""

    def __init__(self, group: str = "TP"):
        self.group = group

    def forward(self, piece):
        n = _size(self.group)
        kg = next(k for k in piece if "gate_proj" in k)
        ku = next(k for k in piece if "up_proj" in k)
        # dim -2 is the output dimension of both [F, H] and stacked-expert [E, F, H] weights
        shards = [torch.cat([piece[kg].chunk(n, -2)[r], piece[ku].chunk(n, -2)[r]], dim=-2) for r in range(n)]
        return {kg.replace("gate_proj", "gate_up_proj"): shards}

    def backward(self, piece):
        (name, shards), = piece.items()
        halves = [s.chunk(2, dim=-2) for s in shards]
        return {name.replace("gate_up_proj", "gate_proj"): torch.cat([h[0] for h in halves], dim=-2),
                name.replace("gate_up_proj", "up_proj"): torch.cat([h[1] for h in halves], dim=-2)}


class UnbindMoE(ReshapeOp):
    """Per-expert HF tensors ``...experts.<i>.<proj>.weight`` <-> one stacked tensor ``[E, ...]`` per proj."""

    def __init__(self, moe_key_prefix: str = "experts."):
        self.prefix = moe_key_prefix
        self._pat = re.compile(re.escape(moe_key_prefix) + r"(\d+)\.")

    def forward(self, piece):
        groups: dict = {}
        for k, t in piece.items():
            m = self._pat.search(k)
            if not m:
                groups.setdefault(k, {})[0] = t
                continue
            groups.setdefault(self._pat.sub(self.prefix, k), {})[int(m.group(1))] = t
        return {k: torch.stack([d[i] for i in sorted(d)]) if len(d) > 1 or self.prefix in k else d[0]
                for k, d in groups.items()}

    def backward(self, piece):
        out = {}
        for k, t in piece.items():
            if self.prefix in k:
                for i, x in enumerate(t.unbind(0)):
                    out[k.replace(self.prefix, f"{self.prefix}{i}.")] = x
            else:
                out[k] = t
        return out


class Script(DataClass):
    """One rule: HF names matching ``src`` (glob / character classes) --``op``--> native ``dst``."""

    src: str = ""
    op: ReshapeOp = None
    dst: str = ""


class OnlineReshaper(ReshapeOp):
    def __init__(self, scripts):
        self.scripts = list(scripts.values()) if isinstance(scripts, dict) else list(scripts)

    @staticmethod
    def get_piece_by_pattern(weights: dict, patterns) -> dict:
        patterns = [patterns] if isinstance(patterns, str) else list(patterns)
        out = {}
        for pat in patterns:
            for k in weights:
                if k == pat or fnmatch.fnmatchcase(k, pat):
                    out[k] = weights[k]
        return out

    def check_forwardable(self) -> None:
        """Every rule names its HF side (``src``): the map can be applied to an HF state dict."""
        missing = [sc for sc in self.scripts if not sc.src]
        if missing:
            raise RuntimeError(f"{len(missing)} reshape rule(s) without .src (first: dst={missing[0].dst!r}): "
                               "the HF names are unknown, so an HF state cannot be mapped in")

    def check_backwardable(self) -> None:
        """Every rule names its native side (``dst``): parameters can be mapped out to HF names."""
        missing = [sc for sc in self.scripts if not sc.dst]
        if missing:
            raise RuntimeError(f"{len(missing)} reshape rule(s) without .dst (first: src={missing[0].src!r}): "
                               "the parameter names are unknown, so nothing can be exported")

    def forward(self, weights: dict) -> dict:
        self.check_forwardable()
        native = {}
        for sc in self.scripts:
            piece = self.get_piece_by_pattern(weights, sc.src)
            if not piece:
                continue
            res = sc.op.forward(piece)
            if len(res) == 1 and "*" not in sc.dst:
                native[sc.dst] = next(iter(res.values()))
            else:
                native.update(res)
        return native

    def backward(self, weights: dict) -> dict:
        self.check_backwardable()
        hf = {}
        for sc in self.scripts:
            if "*" in sc.dst:                      # a rule over a family of parameters
                piece = self.get_piece_by_pattern(weights, sc.dst)
                if piece:
                    hf.update(sc.op.backward(piece))
            elif sc.dst in weights:
                hf.update(sc.op.backward({sc.dst: weights[sc.dst]}))
        return hf


def merge_op_for(param) -> ReshapeOp:
    """How to rebuild the full matrix of a TP-sharded parameter (used by Muon)."""
    if getattr(param, "tensor_model_parallel", False):
        group = getattr(param, "partition_group", "TP")
        if param.partition_dim == 0:
            return Inverse(ColumnParallel(group) + KeepThisTP(group))
        if param.partition_dim == 1:
            return Inverse(RowParallel(group) + KeepThisTP(group))
    return Sequential([])


def build_qwen_reshaper(cfg, layer_ids, first_stage: bool, last_stage: bool) -> OnlineReshaper:
    """HF Qwen3 (dense or MoE) names <-> native names for the layers of one pipeline chunk."""
    scripts = []
    ac = cfg.attn_cfg
    if first_stage:
        scripts.append(Script(src="model.embed_tokens.weight", dst="tok_embeddings.word_embeddings.weight",
                              op=VocabPad(cfg.tok_embed_cfg.vocab_size, 0) + ColumnParallel() + KeepThisTP()
                              + Rename("tok_embeddings.word_embeddings.weight: model.embed_tokens.weight")))
    if last_stage:
        if not cfg.tie_embedding:
            scripts.append(Script(src="lm_head.weight", dst="out_embeddings.output.weight",
                                  op=VocabPad(cfg.out_embed_cfg.vocab_size, 0) + ColumnParallel() + KeepThisTP()
                                  + Rename("out_embeddings.output.weight: lm_head.weight")))
        scripts.append(Script(src="model.norm.weight", dst="out_embeddings.norm.weight",
                              op=Duplicate() + KeepThisTP() + Rename("out_embeddings.norm.weight: model.norm.weight")))
    moe_cfg = getattr(cfg, "moe_cfg", None)
    for i in layer_ids:
        s, d = f"model.layers.{i}", f"layers.{i}"
        scripts.append(Script(src=f"{s}.self_attn.[qkv]_proj.weight", dst=f"{d}.attention.wqkv.weight",
                              op=GQAMergeQKV(ac.num_attention_groups, ac.head_dim or cfg.hidden_size // ac.num_attention_heads)
                              + KeepThisTP() + Rename(f"{d}.attention.wqkv.weight: {s}.self_attn.qkv_proj.weight")))
        if getattr(ac, "use_qkv_bias", False):       # Qwen2-style projections carry a bias on q, k and v
            scripts.append(Script(src=f"{s}.self_attn.[qkv]_proj.bias", dst=f"{d}.attention.wqkv.bias",
                                  op=GQAMergeQKVBias(ac.num_attention_groups, ac.head_dim or cfg.hidden_size // ac.num_attention_heads)
                                  + KeepThisTP() + Rename(f"{d}.attention.wqkv.bias: {s}.self_attn.qkv_proj.bias")))
        scripts.append(Script(src=f"{s}.self_attn.o_proj.weight", dst=f"{d}.attention.wo.weight",
                              op=RowParallel() + KeepThisTP() + Rename(f"{d}.attention.wo.weight: {s}.self_attn.o_proj.weight")))
        for hf_n, nat_n in (("input_layernorm", "attention_norm"), ("post_attention_layernorm", "ffn_norm"),
                            ("self_attn.q_norm", "attention.q_norm"), ("self_attn.k_norm", "attention.k_norm")):
            scripts.append(Script(src=f"{s}.{hf_n}.weight", dst=f"{d}.{nat_n}.weight",
                                  op=Duplicate() + KeepThisTP() + Rename(f"{d}.{nat_n}.weight: {s}.{hf_n}.weight")))
        if moe_cfg is not None and i in moe_cfg.moe_layer_list:
            scripts.append(Script(src=f"{s}.mlp.gate.weight", dst=f"{d}.feed_forward.moe.gate.weight",
                                  op=Duplicate() + KeepThisTP() + Rename(f"{d}.feed_forward.moe.gate.weight: {s}.mlp.gate.weight")))
            scripts.append(Script(src=f"{s}.mlp.experts.*.[gu]*_proj.weight", dst=f"{d}.feed_forward.moe.experts.w1",
                                  op=_ExpertGateUp() + KeepThisEP() + Rename(f"{d}.feed_forward.moe.experts.w1: {s}.mlp.experts.w1")))
            scripts.append(Script(src=f"{s}.mlp.experts.*.down_proj.weight", dst=f"{d}.feed_forward.moe.experts.w2",
                                  op=UnbindMoE("experts.") + KeepThisEP()
                                  + Rename(f"{d}.feed_forward.moe.experts.w2: {s}.mlp.experts.down_proj.weight")))
        else:
            scripts.append(Script(src=f"{s}.mlp.[gu]*_proj.weight", dst=f"{d}.feed_forward.w1.weight",
                                  op=FFNMergeGateUp() + KeepThisTP()
                                  + Rename(f"{d}.feed_forward.w1.weight: {s}.mlp.gate_up_proj.weight")))
            scripts.append(Script(src=f"{s}.mlp.down_proj.weight", dst=f"{d}.feed_forward.w2.weight",
                                  op=RowParallel() + KeepThisTP() + Rename(f"{d}.feed_forward.w2.weight: {s}.mlp.down_proj.weight")))
    return OnlineReshaper(scripts)


class _ExpertGateUp(ReshapeOp):
    """``experts.<i>.gate_proj`` / ``up_proj`` -> stacked ``[E, 2F, H]`` with rows ``[gate | up]``."""

    _pat = re.compile(r"experts\.(\d+)\.(gate|up)_proj")

    def forward(self, piece):
        gates, ups, base = {}, {}, None
        for k, t in piece.items():
            m = self._pat.search(k)
            (gates if m.group(2) == "gate" else ups)[int(m.group(1))] = t
            base = k[: m.start()] + "experts.w1"
        return {base: torch.stack([torch.cat([gates[i], ups[i]], dim=0) for i in sorted(gates)])}

    def backward(self, piece):
        (name, t), = piece.items()
        out = {}
        for i, x in enumerate(t.unbind(0)):
            g, u = x.chunk(2, dim=0)
            out[name.replace("experts.w1", f"experts.{i}.gate_proj.weight")] = g
            out[name.replace("experts.w1", f"experts.{i}.up_proj.weight")] = u
        return out
