"""MoE kernel micro-benchmarks on one GPU: routing index, row scatter / weighted gather, grouped GEMM and
the routed SwiGLU FFN, each checked against its plain PyTorch statement before it is timed.

Workloads follow the reference's benchmark definitions (``benchmarks/benchmark_moe_routing.py:15-36``,
``benchmark_grouped_gemm.py:15-26``, ``benchmark_routed_grouped_ffn.py:15-28``) plus the Qwen3-30B-A3B layer
shape (8192 tokens, H=2048, 128 experts, F=768, top-8).  Bandwidth-bound cases report the fraction of the
measured copy bandwidth, GEMM-bound cases the fraction of the measured bf16 GEMM peak.

    python benchmarks/benchmark_moe.py [--only routing,router,movers,grouped_gemm,routed_ffn] [--json out.json]
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from benchmarks.common import measured_peaks, time_cuda  # noqa: E402
from steptronoss_b200.ops import moe, native  # noqa: E402
from steptronoss_b200.ops.grouped import grouped_gemm_reduce, grouped_gemm_rows  # noqa: E402


def _ids(T, E, K, invalid=0.0, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    ids = torch.rand(T, E, device="cuda", generator=g).topk(K, dim=1).indices
    if invalid:
        ids = torch.where(torch.rand(T, K, device="cuda", generator=g) < invalid, torch.full_like(ids, -1), ids)
    return ids


def _emit(rows, **row):
    rows.append(row)
    print(json.dumps(row), flush=True)


def bench_routing(rows, peaks):
    for T, E, K in ((8192, 128, 2), (32768, 288, 2), (8192, 128, 8)):
        ids = _ids(T, E, K, 0.1)
        plan = moe.RoutePlan(ids, E)
        dest, offsets, counts = moe.index_compute(ids, E)
        assert torch.equal(plan.dest, dest) and torch.equal(plan.offsets, offsets) and torch.equal(plan.counts, counts)
        t_native = time_cuda(lambda: moe.RoutePlan(ids, E), flush=False)

        def torch_path():
            d, o, _ = moe.index_compute(ids, E)
            moe.tile_groups_from_offsets(o, plan.rows)
            moe.slot_of_row_from_dest(d, plan.rows)

        t_torch = time_cuda(torch_path, flush=False)
        _emit(rows, bench="routing_index", tokens=T, experts=E, top_k=K, native_ms=t_native["best_ms"],
              torch_ops_ms=t_torch["best_ms"], speedup=t_torch["best_ms"] / t_native["best_ms"])


def bench_router(rows, peaks):
    for T, E, K, sigmoid in ((8192, 128, 2, False), (32768, 288, 2, False), (8192, 128, 8, False), (8192, 288, 8, True)):
        logits = (torch.randn(T, E, device="cuda") * 2).requires_grad_()
        bias = torch.zeros(E, device="cuda") if sigmoid else None
        gw, gps = torch.randn(T, K, device="cuda"), torch.randn(E, device="cuda")
        res = {}
        for name, fn in (("native", moe.fused_router), ("torch_ops", moe.router_reference)):
            def fwd():
                return fn(logits, bias, K, sigmoid, True, 1e-20 if sigmoid else 0.0)

            def fwd_bwd():
                _ids, w, ps, _h, _s = fwd()
                torch.autograd.grad((w * gw).sum() + (ps * gps).sum(), logits)

            res[name] = (time_cuda(fwd, flush=False)["best_ms"], time_cuda(fwd_bwd, flush=False)["best_ms"])
        _emit(rows, bench="router", tokens=T, experts=E, top_k=K, sigmoid=sigmoid, native_fwd_ms=res["native"][0],
              native_fwd_bwd_ms=res["native"][1], torch_ops_fwd_ms=res["torch_ops"][0],
              torch_ops_fwd_bwd_ms=res["torch_ops"][1], speedup_fwd_bwd=res["torch_ops"][1] / res["native"][1])


def bench_movers(rows, peaks):
    for T, E, K, H in ((8192, 128, 8, 2048), (8192, 36, 2, 4096)):
        ids = _ids(T, E, K)
        plan = moe.RoutePlan(ids, E)
        used = int(plan.offsets[-1])
        x = torch.randn(T, H, device="cuda").to(torch.bfloat16)
        y = torch.randn(plan.rows, H, device="cuda").to(torch.bfloat16)
        w = torch.rand(T, K, device="cuda")
        g_rows = torch.randn(plan.rows, H, device="cuda").to(torch.bfloat16)
        g_tok = torch.randn(T, H, device="cuda").to(torch.bfloat16)
        row_b = H * 2
        cases = {
            # name: (native fn, torch fn, algorithmic bytes)
            "scatter": (lambda: moe.moe_scatter(x, plan.dest, plan.rows, plan),
                        lambda: moe.moe_scatter(x, plan.dest, plan.rows), (T * K + used) * row_b),
            "gather": (lambda: moe.moe_weighted_gather(y, plan.dest, w, plan),
                       lambda: moe.moe_weighted_gather(y, plan.dest, w), (T * K + T) * row_b),
        }
        for name, (fn, ref, nbytes) in cases.items():
            a, b = fn(), ref()
            n = used if name == "scatter" else T
            err = float((a[:n].float() - b[:n].float()).abs().max())
            assert err < 0.05, (name, err)
            tn, tt = time_cuda(fn), time_cuda(ref)
            gbs = nbytes / (tn["best_ms"] * 1e-3) / 1e9
            _emit(rows, bench=name, tokens=T, experts=E, top_k=K, hidden=H, native_ms=tn["best_ms"],
                  torch_ops_ms=tt["best_ms"], gb_per_s=gbs, frac_of_measured_copy=gbs / peaks["hbm_gbs"])
        # backward passes
        xg, yg, wg = x.clone().requires_grad_(), y.clone().requires_grad_(), w.clone().requires_grad_()
        for name, build, grads, gin, nbytes in (
            ("scatter_bwd", lambda p: moe.moe_scatter(xg, plan.dest, plan.rows, p), [xg], g_rows, (T * K + T) * row_b),
            ("gather_bwd", lambda p: moe.moe_weighted_gather(yg, plan.dest, wg, p), [yg, wg], g_tok,
             (2 * T * K + T + (used - T * K)) * row_b),
        ):
            out_n, out_t = build(plan), build(None)
            fn = lambda: torch.autograd.grad(out_n, grads, gin, retain_graph=True)  # noqa: E731
            ref = lambda: torch.autograd.grad(out_t, grads, gin, retain_graph=True)  # noqa: E731
            tn, tt = time_cuda(fn), time_cuda(ref)
            gbs = nbytes / (tn["best_ms"] * 1e-3) / 1e9
            _emit(rows, bench=name, tokens=T, experts=E, top_k=K, hidden=H, native_ms=tn["best_ms"],
                  torch_ops_ms=tt["best_ms"], gb_per_s=gbs, frac_of_measured_copy=gbs / peaks["hbm_gbs"])
        del x, y, g_rows, g_tok, xg, yg
        torch.cuda.empty_cache()


def bench_grouped_gemm(rows, peaks):
    for G, per, K, N in ((36, 3256, 4096, 2560), (128, 512, 2048, 1536)):
        seg = (per + 127) // 128 * 128
        M = G * seg
        offsets = (torch.arange(G + 1, device="cuda", dtype=torch.int32) * seg)
        x = torch.zeros(M, K, device="cuda", dtype=torch.bfloat16)
        gy = torch.zeros(M, N, device="cuda", dtype=torch.bfloat16)
        for g in range(G):  # real rows random, padding rows zero
            x[g * seg:g * seg + per].normal_()
            gy[g * seg:g * seg + per].normal_()
        w = (torch.randn(G, N, K, device="cuda") * 0.02).to(torch.bfloat16)
        tg = moe.tile_groups_from_offsets(offsets, M)
        y = grouped_gemm_rows(x, w, offsets, tile_group=tg)
        ref = torch.einsum("gmk,gnk->gmn", x.view(G, seg, K)[:4].float(), w[:4].float())
        err = float((y.view(G, seg, N)[:4].float() - ref).abs().max() / ref.abs().max())
        assert err < 2e-2, err
        flops = 2.0 * G * per * K * N
        for name, fn in (("fwd", lambda: grouped_gemm_rows(x, w, offsets, tile_group=tg)),
                         ("dgrad", lambda: grouped_gemm_rows(gy, w, offsets, trans_b=False, tile_group=tg)),
                         ("wgrad", lambda: grouped_gemm_reduce(gy, x, offsets, G))):
            t = time_cuda(fn)
            tf = flops / (t["best_ms"] * 1e-3) / 1e12
            _emit(rows, bench="grouped_gemm_" + name, groups=G, rows_per_group=per, K=K, N=N, best_ms=t["best_ms"],
                  tflops_useful=tf, frac_of_measured_peak=tf / peaks["bf16_tflops"])
        del x, gy, w, y
        torch.cuda.empty_cache()


def bench_routed_ffn(rows, peaks):
    for T, H, E, F, K, invalid in ((8192, 4096, 36, 1280, 2, 0.1), (8192, 2048, 128, 768, 8, 0.0)):
        ids = _ids(T, E, K, invalid)
        x = torch.randn(T, H, device="cuda").to(torch.bfloat16).requires_grad_()
        w = torch.rand(T, K, device="cuda")
        w1 = (torch.randn(E, 2 * F, H, device="cuda") * 0.02).to(torch.bfloat16).requires_grad_()
        w2 = (torch.randn(E, H, F, device="cuda") * 0.02).to(torch.bfloat16).requires_grad_()
        out = moe.routed_grouped_ffn(x, ids, w, w1, w2)
        with torch.no_grad():
            ref = moe.routed_grouped_ffn_reference(x[:512].float(), ids[:512], w[:512], w1.float(), w2.float())
        err = float((out[:512].float() - ref).abs().max() / ref.abs().max())
        assert err < 3e-2, err
        gout = torch.randn_like(out)
        slots = float((ids >= 0).sum())
        flops_f = 2.0 * slots * H * 3 * F
        tf = time_cuda(lambda: moe.routed_grouped_ffn(x, ids, w, w1, w2))

        def fwd_bwd():
            o = moe.routed_grouped_ffn(x, ids, w, w1, w2)
            torch.autograd.grad(o, [x, w1, w2], gout)

        tb = time_cuda(fwd_bwd)
        _emit(rows, bench="routed_ffn", tokens=T, hidden=H, experts=E, ffn=F, top_k=K, invalid=invalid,
              fwd_ms=tf["best_ms"], fwd_bwd_ms=tb["best_ms"],
              fwd_tflops=flops_f / (tf["best_ms"] * 1e-3) / 1e12,
              fwd_bwd_tflops=3 * flops_f / (tb["best_ms"] * 1e-3) / 1e12,
              fwd_bwd_frac_of_measured_peak=3 * flops_f / (tb["best_ms"] * 1e-3) / 1e12 / peaks["bf16_tflops"])
        del x, w1, w2, out
        torch.cuda.empty_cache()


BENCHES = {"routing": bench_routing, "router": bench_router, "movers": bench_movers, "grouped_gemm": bench_grouped_gemm,
           "routed_ffn": bench_routed_ffn}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--only", default=None)
    ap.add_argument("--json", default=None)
    args = ap.parse_args()
    peaks = measured_peaks()
    rows = []
    for name, fn in BENCHES.items():
        if args.only and name not in args.only.split(","):
            continue
        fn(rows, peaks)
        torch.cuda.synchronize()
        native.raise_if_kernel_error()
    if args.json:
        json.dump({"peaks": peaks, "rows": rows}, open(args.json, "w"), indent=1)


if __name__ == "__main__":
    main()
