"""Worker (torch.distributed.run, one rank per GPU): Muon's gather of tensor-parallel shards over peer memory gives
the matrix that the NCCL all-gather gives, for row-split, column-split and block-interleaved parameters."""
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402


def main():
    from steptronoss_b200.exp.base_exp import ParallelConfig
    from steptronoss_b200.ops import native
    from steptronoss_b200.optim import muon
    from steptronoss_b200.parallel.state import PM

    PM.initialize()
    mesh = ParallelConfig()
    mesh.tensor_model_parallel_size = PM.world_size
    mesh.expert_tensor_parallel_size = 1
    PM.set_mesh(mesh)
    dev = torch.device("cuda", torch.cuda.current_device())
    g = torch.Generator(device=dev).manual_seed(5 + PM.world_rank)
    res = {}
    cases = {"rows": (0, None, (256, 512)), "cols": (1, None, (384, 128)), "blocks": (0, [512, 256], (384, 256))}
    for name, (dim, blocks, shape) in cases.items():
        shard = torch.randn(shape, device=dev, generator=g).to(torch.bfloat16)

        class P:  # what gather_full_matrix reads from a parameter
            tensor_model_parallel, partition_dim, partition_group = True, dim, "TP"
            partition_blocks = blocks

        full_peer = muon.gather_full_matrix(shard, P).clone()
        used_peer = muon._gather_over_peer_memory(shard, dim, "TP", PM.world_size) is not None
        os.environ["STB200_PEER_TP"] = "0"
        parts = [torch.empty_like(shard) for _ in range(PM.world_size)]
        dist.all_gather(parts, shard.contiguous(), group=PM.group_of("TP"))
        if blocks:
            per = [b // PM.world_size for b in blocks]
            pieces = [p.split(per, dim=dim) for p in parts]
            want = torch.cat([torch.cat([pieces[r][i] for r in range(PM.world_size)], dim=dim) for i in range(len(blocks))], dim=dim)
        else:
            want = torch.cat(parts, dim=dim)
        assert full_peer.shape == want.shape and torch.equal(full_peer, want), name
        back = muon.slice_own_shard(full_peer, P)
        assert torch.equal(back, shard), name
        res[name] = bool(used_peer)
    torch.cuda.synchronize()
    native.raise_if_kernel_error()
    dist.barrier()
    if PM.world_rank == 0:
        print("RESULT " + json.dumps(res), flush=True)


if __name__ == "__main__":
    main()
