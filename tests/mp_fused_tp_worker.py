"""Worker for the fused GEMM+collective tests (launched by torch.distributed.run, one rank per GPU).

Checks ``all_gather_gemm`` and ``gemm_reduce_scatter`` against fp32 PyTorch restatements built from NCCL
collectives, over several calls (slot reuse, buffer growth), both weight layouts, and a bounded-wait case
in which one rank stays away from a call.  Prints one ``RESULT`` JSON line from rank 0.
"""
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402


def _ref_ag_gemm(x, w, b_mn, group):
    tp = dist.get_world_size(group)
    full = torch.empty((x.shape[0] * tp, x.shape[1]), dtype=x.dtype, device=x.device)
    dist.all_gather_into_tensor(full, x.contiguous(), group=group)
    wm = w.float() if b_mn else w.float().t()
    return full.float() @ wm, full


def _ref_gemm_rs(a, w, b_mn, group):
    tp = dist.get_world_size(group)
    wm = w.float() if b_mn else w.float().t()
    part = (a.float() @ wm).to(torch.bfloat16).float()  # partial products travel as bf16
    out = torch.empty((a.shape[0] // tp, part.shape[1]), dtype=torch.float32, device=a.device)
    dist.reduce_scatter_tensor(out, part, group=group)
    return out


def main():
    mode = sys.argv[1] if len(sys.argv) > 1 else "check"
    from steptronoss_b200.ops import native
    from steptronoss_b200.parallel import symm
    from steptronoss_b200.parallel.state import PM

    PM.initialize()
    PM.new_parallel("TP", [list(range(PM.world_size))])
    group = PM.group_of("TP")
    rank, tp = PM.rank_in("TP"), PM.size_of("TP")
    dev = torch.device("cuda", torch.cuda.current_device())
    assert symm.enabled("TP"), "peer-memory arena could not be created"
    res = {"max_err": {}}
    g = torch.Generator(device=dev).manual_seed(1234 + rank)

    # (rows per rank, K, N); the last two exercise rows wider than one 32 KB communication unit and a 4-row unit
    shapes = [(256, 512, 768), (384, 1024, 512), (256, 512, 768), (1024, 2048, 2304), (128, 256, 256),
              (128, 16896, 256), (256, 4096, 4096)]
    for it, (rows, k, n) in enumerate(shapes):
        for b_mn in (False, True):
            x = torch.randn(rows, k, device=dev, generator=g).to(torch.bfloat16)
            if it % 2 == 1:   # rows with a pitch: the communication units are loaded row by row
                x = torch.randn(rows, k + 64, device=dev, generator=g).to(torch.bfloat16)[:, :k]
            w = (torch.randn((k, n) if b_mn else (n, k), device=dev, generator=g) * 0.05).to(torch.bfloat16)
            dist.broadcast(w, src=dist.get_global_rank(group, 0), group=group)
            y, full = symm.all_gather_gemm(x, w, "TP", b_mn_major=b_mn)
            y_ref, full_ref = _ref_ag_gemm(x, w, b_mn, group)
            assert torch.equal(full, full_ref), f"gathered rows differ (call {it}, b_mn={b_mn})"
            err = float((y.float() - y_ref).abs().max() / y_ref.abs().max())
            res["max_err"][f"ag_{rows}x{k}x{n}_{int(b_mn)}_{it}"] = err
            assert err < 1e-2, (rows, k, n, b_mn, err)
            # gather only
            _, full2 = symm.all_gather_gemm(x, None, "TP")
            assert torch.equal(full2, full_ref)
            # reduce-scatter: A is [tp*rows, k]
            a = torch.randn(rows * tp, k, device=dev, generator=g).to(torch.bfloat16)
            out = symm.gemm_reduce_scatter(a, w, "TP", b_mn_major=b_mn)
            out_ref = _ref_gemm_rs(a, w, b_mn, group)
            err = float((out.float() - out_ref).abs().max() / out_ref.abs().max())
            res["max_err"][f"rs_{rows}x{k}x{n}_{int(b_mn)}_{it}"] = err
            assert err < 1e-2, (rows, k, n, b_mn, err)
    torch.cuda.synchronize()
    native.raise_if_kernel_error()

    # run-to-run determinism of the reduction
    a = torch.randn(512 * tp, 1024, device=dev, generator=g).to(torch.bfloat16)
    w = (torch.randn(512, 1024, device=dev, generator=g) * 0.05).to(torch.bfloat16)
    o1 = symm.gemm_reduce_scatter(a, w, "TP")
    o2 = symm.gemm_reduce_scatter(a, w, "TP")
    assert torch.equal(o1, o2)

    if mode == "timeout":
        # One rank stays away from a call: the others' waits run out, the kernel reports it in the status word
        # and returns; the context stays usable and the next call (all ranks present) is correct.
        ar = symm.arena("TP")
        old = symm._WAIT_NS
        symm._WAIT_NS = int(0.3e9)
        x = torch.randn(256, 512, device=dev, generator=g).to(torch.bfloat16)
        torch.cuda.synchronize()
        dist.barrier()
        if rank == 0:
            symm.all_gather_gemm(x, None, "TP")
            torch.cuda.synchronize()
            code = int(native.status_word(dev).item())
            native.status_word(dev).zero_()
            res["timeout_code"] = code
            assert code == 5, code
        else:
            ar.ag_epoch += 1  # keep the call numbering aligned with the rank that did call
        symm._WAIT_NS = old
        torch.cuda.synchronize()
        dist.barrier()
        _, full = symm.all_gather_gemm(x, None, "TP")
        ref = torch.empty_like(full)
        dist.all_gather_into_tensor(ref, x, group=group)
        assert torch.equal(full, ref)
        native.raise_if_kernel_error()

    torch.cuda.synchronize()
    dist.barrier()
    if rank == 0:
        print("RESULT " + json.dumps(res), flush=True)
    symm.shutdown()
    dist.barrier()


if __name__ == "__main__":
    main()
