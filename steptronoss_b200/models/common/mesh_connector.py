"""Move batch-shaped tensors between two static parallel meshes of the same job.

Reference: ``steptronoss/model/common/mesh_connector.py:43-371``.  Used when an auxiliary module runs under
another mesh than its caller, e.g. text ranks (TP=8) handing raw images to a vision encoder that runs data
parallel over the same 8 GPUs, and getting the encoded features back.

Model.  A mesh is seen as *replicas* (the data-parallel coordinate that remains after removing PP, CP and
TP); transfers never leave a replica.  ``dup_dim`` names the dimensions along which ranks hold identical
payloads; dropping them from a rank's coordinates gives its *node*, the ranks of one node form a duplicate
group and its first rank is the leader.

* ``forward(t)``: in every replica the canonical source node's leader cuts ``t`` along dim 0 into one shard
  per destination node and sends each shard to that node's leader, which fans it out to its duplicates.
* ``backward(t)``: every destination leader sends its tensor to the leaders of all source nodes of the
  replica, which concatenate the shards in order and fan the result out to their duplicates.

Payloads travel as tensors (batched ``isend``/``irecv`` on the job's default group, NCCL on GPUs) after one
small object all-gather that tells every receiver what to expect; the reference pickles the tensors into an
object all-to-all.  Every rank must call ``forward`` / ``backward`` in the same sequence, with an empty tensor
when it has nothing to send.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist

from ...parallel.state import PM

_DIMS = ("PP", "CP", "TP")


@dataclass(frozen=True)
class _Node:
    replica: int
    pp: int | None
    cp: int | None
    tp: int | None

    def key(self):
        return (self.replica, -1 if self.pp is None else self.pp, -1 if self.cp is None else self.cp,
                -1 if self.tp is None else self.tp)


@dataclass(frozen=True)
class _ShardMeta:
    batch_size: int
    shard_count: int
    shard_id: int

    def bounds(self) -> tuple[int, int]:
        base, extra = divmod(self.batch_size, self.shard_count)
        start = self.shard_id * base + min(self.shard_id, extra)
        return start, min(start + base + (1 if self.shard_id < extra else 0), self.batch_size)


class _Mesh:
    """Coordinates, nodes and duplicate groups of every rank under one ParallelConfig."""

    def __init__(self, cfg, world: int, dup_dim: tuple, make_groups: bool):
        pp, cp, tp = (int(cfg.pipeline_model_parallel_size), int(cfg.context_parallel_size),
                      int(cfg.tensor_model_parallel_size))
        mp = pp * cp * tp
        if mp <= 0 or world % mp:
            raise ValueError(f"MeshConnector requires WORLD_SIZE to be divisible by PP*CP*TP, got world_size={world}, "
                             f"PP={pp}, CP={cp}, TP={tp}")
        with PM.use_mesh(cfg):
            fam = {d: PM.world_ranks_of(d) for d in _DIMS}
        self.node_of: dict[int, _Node] = {}
        self.pos: dict[int, dict] = {}
        for r in range(world):
            pos = {d: next(g.index(r) for g in fam[d] if r in g) for d in _DIMS}
            replica = (r // (cp * tp)) % (world // mp)
            self.node_of[r] = _Node(replica, *(None if d in dup_dim else pos[d] for d in _DIMS))
            self.pos[r] = pos
        self.members: dict[_Node, list[int]] = {}
        for r, n in self.node_of.items():
            self.members.setdefault(n, []).append(r)
        for n, ranks in self.members.items():
            ranks.sort(key=lambda r: tuple(self.pos[r][d] for d in dup_dim))
        self.groups: dict[_Node, object] = {}
        if make_groups:  # collective: every rank creates every group, in the same order
            for n in sorted(self.members, key=_Node.key):
                m = self.members[n]
                self.groups[n] = dist.new_group(m) if len(m) > 1 else None

    def leader(self, node: _Node) -> int:
        return self.members[node][0]

    def nodes_of_replica(self, replica: int) -> list:
        return sorted((n for n in self.members if n.replica == replica), key=_Node.key)


class MeshConnector:
    def __init__(self, src_mesh, dst_mesh, *, is_data_source: bool, dup_dim=("TP",)):
        self.dup_dim = tuple(d.upper() for d in dup_dim)
        if len(set(self.dup_dim)) != len(self.dup_dim):
            raise ValueError(f"MeshConnector dup_dim contains duplicates: {self.dup_dim}")
        bad = sorted(set(self.dup_dim) - set(_DIMS))
        if bad:
            raise ValueError(f"MeshConnector dup_dim only supports {_DIMS}, got unsupported dims {bad}")
        self.world, self.rank = PM.world_size, PM.world_rank
        multi = self.world > 1 and dist.is_initialized()
        self.src = _Mesh(src_mesh, self.world, self.dup_dim, multi)
        self.dst = _Mesh(dst_mesh, self.world, self.dup_dim, multi)
        flags = [is_data_source]
        if multi:
            flags = [None] * self.world
            dist.all_gather_object(flags, is_data_source)
        self.source_nodes = {self.src.node_of[r] for r, f in enumerate(flags) if f}
        self.canonical: dict[int, _Node] = {}
        for n in sorted(self.source_nodes, key=_Node.key):
            self.canonical.setdefault(n.replica, n)
        self._last_meta: _ShardMeta | None = None

    # ------------------------------------------------------------------ plumbing
    def _device(self):
        if torch.cuda.is_available() and dist.is_initialized() and dist.get_backend() == "nccl":
            return torch.device("cuda", torch.cuda.current_device())
        return torch.device("cpu")

    def _exchange(self, sends: dict) -> dict:
        """``sends[dst_rank] = (tensor, meta)`` -> ``{src_rank: (tensor, meta)}`` on the receivers."""
        if self.world == 1 or not dist.is_initialized():
            return {self.rank: v for d, v in sends.items() if d == self.rank}
        dev = self._device()
        notice = {d: (tuple(t.shape), str(t.dtype).split(".")[-1], m) for d, (t, m) in sends.items()}
        all_notices = [None] * self.world
        dist.all_gather_object(all_notices, notice)
        ops, recv, keep = [], {}, []
        for d, (t, _m) in sorted(sends.items()):
            if d == self.rank:
                continue
            buf = t.to(dev).contiguous()
            keep.append(buf)
            if buf.numel():
                ops.append(dist.P2POp(dist.isend, buf, d))
        for s in range(self.world):
            n = all_notices[s].get(self.rank)
            if n is None:
                continue
            shape, dtype, meta = n
            if s == self.rank:
                recv[s] = (sends[self.rank][0], meta)
                continue
            buf = torch.empty(shape, dtype=getattr(torch, dtype), device=dev)
            recv[s] = (buf, meta)
            if buf.numel():
                ops.append(dist.P2POp(dist.irecv, buf, s))
        for w in (dist.batch_isend_irecv(ops) if ops else []):
            w.wait()
        return recv

    def _fanout(self, payload, mesh: _Mesh, node: _Node):
        members, group = mesh.members[node], mesh.groups.get(node)
        if len(members) == 1 or group is None:
            return payload
        leader = members[0]
        head = [None]
        if self.rank == leader:
            head = [None if payload is None else (tuple(payload[0].shape), str(payload[0].dtype).split(".")[-1], payload[1])]
        dist.broadcast_object_list(head, src=leader, group=group)
        if head[0] is None:
            return None
        shape, dtype, meta = head[0]
        dev = self._device()
        t = payload[0].to(dev).contiguous() if self.rank == leader else torch.empty(shape, dtype=getattr(torch, dtype), device=dev)
        if t.numel():
            dist.broadcast(t, src=leader, group=group)
        return t, meta

    # ------------------------------------------------------------------ API
    def forward(self, data: torch.Tensor | None) -> torch.Tensor | None:
        my_src = self.src.node_of[self.rank]
        sender = (data is not None and self.rank == self.src.leader(my_src)
                  and self.canonical.get(my_src.replica) == my_src)
        sends = {}
        if sender:
            nodes = self.dst.nodes_of_replica(my_src.replica)
            for i, n in enumerate(nodes):
                meta = _ShardMeta(int(data.shape[0]), len(nodes), i)
                a, b = meta.bounds()
                sends[self.dst.leader(n)] = (data[a:b].contiguous(), meta)
        got = self._exchange(sends)
        my_dst = self.dst.node_of[self.rank]
        payload = next(iter(got.values()), None) if self.rank == self.dst.leader(my_dst) else None
        payload = self._fanout(payload, self.dst, my_dst)
        if payload is None:
            self._last_meta = None
            return None
        self._last_meta = payload[1]
        return payload[0]

    def backward(self, data: torch.Tensor | None) -> torch.Tensor | None:
        # a rank that received nothing in forward() still takes part in the exchange (it is collective)
        if data is not None and self._last_meta is None:
            raise RuntimeError("MeshConnector.backward() called before forward().")
        my_dst = self.dst.node_of[self.rank]
        sends = {}
        if data is not None and self.rank == self.dst.leader(my_dst):
            for n in sorted((s for s in self.source_nodes if s.replica == my_dst.replica), key=_Node.key):
                sends[self.src.leader(n)] = (data, self._last_meta)
        got = self._exchange(sends)
        my_src = self.src.node_of[self.rank]
        restored = None
        if self.rank == self.src.leader(my_src) and got:
            parts = sorted(got.values(), key=lambda p: p[1].shard_id)
            dev = data.device if data is not None else parts[0][0].device
            shards = [t.to(dev) for t, _ in parts if t.shape[0] > 0]
            total = parts[0][1].batch_size
            out = (torch.cat(shards, dim=0)[:total].contiguous() if shards
                   else parts[0][0].new_empty((0, *parts[0][0].shape[1:])))
            restored = (out, parts[0][1])
        restored = self._fanout(restored, self.src, my_src)
        return None if restored is None else restored[0]
