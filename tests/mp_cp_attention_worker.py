"""Worker (torch.distributed.run, one rank per GPU, CP = world size): context-parallel attention whose kernels address
the gathered keys by global position, against (a) the packed-keys statement over NCCL and (b) fp32 attention over
the whole sequence, forward and backward, for packed documents that start off the 128-row grid, span several
chunks, and leave a padded tail."""
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402


def main():
    from steptronoss_b200.exp.base_exp import ParallelConfig
    from steptronoss_b200.ops import native
    from steptronoss_b200.ops.attention import attention_reference
    from steptronoss_b200.parallel import context_parallel as cpm
    from steptronoss_b200.parallel.state import PM

    PM.initialize()
    mesh = ParallelConfig()
    mesh.context_parallel_size = PM.world_size
    PM.set_mesh(mesh)
    cp, rank = PM.size_of("CP"), PM.rank_in("CP")
    dev = torch.device("cuda", torch.cuda.current_device())
    hq, hkv, D = 4, 2, 128
    res = {}
    cases = {
        "one_doc": (2048 * cp, None),
        "docs_off_grid": (1024 * cp, [0, 100, 611, 1300, 1024 * cp - 90]),       # last 90 rows: padding
        "long_and_short": (4096 * cp, [0, 37, 5000 if cp == 2 else 9000, 4096 * cp]),
    }
    for name, (total, cu) in cases.items():
        g = torch.Generator(device=dev).manual_seed(11)          # the same full tensors on every rank
        full = [torch.randn(total, h, D, device=dev, generator=g).to(torch.bfloat16) for h in (hq, hkv, hkv)]
        dout_full = torch.randn(total, hq, D, device=dev, generator=g).to(torch.bfloat16)
        cu_t = None if cu is None else torch.tensor(cu, dtype=torch.int32, device=dev)
        meta = cpm.build_cp_meta(cu_t, total, device=dev)
        local = [cpm.scatter_to_balanced_cp_region(t).clone().requires_grad_(True) for t in full]
        dout = cpm.scatter_to_balanced_cp_region(dout_full)

        def run(peer: bool):
            cpm.PEER_PATH = peer
            for t in local:
                t.grad = None
            out = cpm.cp_attention(*local, meta, causal=True)
            out.backward(dout)
            return [out.detach().float()] + [t.grad.float().clone() for t in local]

        got = run(True)
        assert cpm._peer_path_ok(*local, meta), "peer path was not taken"
        packed = run(False)
        # fp32 statement on the whole sequence; documents after the last boundary attend to themselves only
        ref_in = [t.float().requires_grad_(True) for t in full]
        cu_ref = cu_t
        if cu is not None and cu[-1] < total:
            cu_ref = torch.tensor(cu + [total], dtype=torch.int32, device=dev)
        ref_out = attention_reference(*ref_in, cu_ref, cu_ref, causal=True)
        ref_out.backward(dout_full.float())
        want = [cpm.scatter_to_balanced_cp_region(t) for t in (ref_out.detach(), *(t.grad for t in ref_in))]
        for label, a, b, c in zip(("o", "dq", "dk", "dv"), got, packed, want):
            scale = float(c.abs().max()) + 1e-6
            res[f"{name}_{label}_vs_fp32"] = float((a - c).abs().max()) / scale
            res[f"{name}_{label}_vs_packed"] = float((a - b).abs().max()) / scale
    torch.cuda.synchronize()
    native.raise_if_kernel_error()
    worst = torch.tensor([max(res.values())], device=dev)
    dist.all_reduce(worst, op=dist.ReduceOp.MAX)
    res["worst_over_ranks"] = float(worst.item())
    dist.barrier()
    if PM.world_rank == 0:
        print("RESULT " + json.dumps(res), flush=True)
    from steptronoss_b200.parallel import symm

    symm.shutdown()


if __name__ == "__main__":
    main()
