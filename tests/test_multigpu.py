"""Multi-GPU training through the native kernels: TP(+SP), DP ZeRO-1, CP and PP layouts on 2 GPUs must
reproduce the 1-GPU loss curve within bf16 tolerance."""
import json
import os
import subprocess
import sys

import pytest

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BASE = dict(gbs=4, seq=512, iters=3, layers=2, hidden=512, heads=4, kv_heads=2, head_dim=128, ffn=1024, vocab=2048,
            min_doc=32, max_doc=256)


def _launch(nproc: int, kw: dict, steps: int = 3, port: int = 29611, extra_env: dict | None = None):
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", **(extra_env or {}))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(ROOT, "tests", "mp_gpu_worker.py"),
           json.dumps(kw), str(steps)]
    if nproc == 1:
        cmd = [sys.executable, os.path.join(ROOT, "tests", "mp_gpu_worker.py"), json.dumps(kw), str(steps)]
        env.pop("WORLD_SIZE", None)
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=400, env=env, cwd=ROOT)
    assert out.returncode == 0, out.stdout[-3000:] + out.stderr[-3000:]
    line = [l for l in out.stdout.splitlines() if l.startswith("RESULT ")][-1]
    return json.loads(line[len("RESULT "):])


@pytest.fixture(scope="module")
def single():
    return _launch(1, dict(BASE))


@pytest.mark.parametrize("layout", [dict(tp=2, sp=True), dict(tp=2, sp=False), dict(), dict(cp=2), dict(pp=2)],
                         ids=["tp2_sp", "tp2", "dp2_zero1", "cp2", "pp2"])
def test_two_gpu_layout_matches_one_gpu(single, layout):
    res = _launch(2, dict(BASE, **layout), port=29620 + len(str(layout)) % 50)
    for a, b in zip(res["losses"], single["losses"]):
        assert abs(a - b) < 3e-2 * abs(b), (layout, res["losses"], single["losses"])


def test_zero1_over_peer_memory_equals_the_nccl_statement():
    """dp2: reduce + Adam + parameter refresh through peer memory gives the loss curve and gradient norms of the
    reduce-scatter / all-gather path (the gradient sums are identical; the squared norm is added up in another
    order, so the clip coefficient and what follows agree to fp32 rounding)."""
    peer = _launch(2, dict(BASE), steps=5, port=29671, extra_env={"STB200_PEER_ZERO": "1"})
    nccl = _launch(2, dict(BASE), steps=5, port=29672, extra_env={"STB200_PEER_ZERO": "0"})
    assert peer["peer_zero_groups"] == ["DP"] and nccl["peer_zero_groups"] == []
    for a, b in zip(peer["losses"], nccl["losses"]):
        assert abs(a - b) <= 5e-5 * max(1.0, abs(b)), (peer["losses"], nccl["losses"])
    for a, b in zip(peer["grad_norms"], nccl["grad_norms"]):
        assert abs(a - b) <= 1e-3 * max(1.0, abs(b)), (peer["grad_norms"], nccl["grad_norms"])


def _launch_fused(nproc: int, mode: str, port: int):
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(port),
           os.path.join(ROOT, "tests", "mp_fused_tp_worker.py"), mode]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=400, env=env, cwd=ROOT)
    assert out.returncode == 0, out.stdout[-3000:] + out.stderr[-3000:]
    line = [l for l in out.stdout.splitlines() if l.startswith("RESULT ")][-1]
    return json.loads(line[len("RESULT "):])


def test_fused_gemm_collectives_match_nccl_statement():
    """all-gather->GEMM and GEMM->reduce-scatter over peer memory against NCCL + fp32 matmul on 2 GPUs."""
    res = _launch_fused(2, "check", 29701)
    assert res["max_err"] and max(res["max_err"].values()) < 1e-2


def test_fused_gemm_collectives_match_nccl_statement_on_four_gpus():
    """The same check at TP=4, the degree of the 8-GPU headline layout (three peers per push, four partial copies
    per reduced tile)."""
    import torch

    if torch.cuda.device_count() < 4:
        pytest.skip("needs >= 4 CUDA devices")
    res = _launch_fused(4, "check", 29703)
    assert res["max_err"] and max(res["max_err"].values()) < 1e-2


def test_fused_gemm_collective_wait_runs_out_without_hanging():
    """A rank that stays away from one call: the peer's bounded wait reports code 5, the next call works."""
    res = _launch_fused(2, "timeout", 29702)
    assert res["timeout_code"] == 5


def test_peer_memory_moe_dispatcher_matches_all_to_all():
    """Dispatch / combine over peer memory against the NCCL all-to-all statement on 2 GPUs (forward, backward)."""
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29731", os.path.join(ROOT, "tests", "mp_peer_dispatch_worker.py")]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=400, env=env, cwd=ROOT)
    assert out.returncode == 0, out.stdout[-3000:] + out.stderr[-3000:]
    res = json.loads([l for l in out.stdout.splitlines() if l.startswith("RESULT ")][-1][len("RESULT "):])
    assert max(v for k, v in res.items() if not k.startswith("ms_")) < 2e-2


def test_expert_parallel_moe_block_peer_vs_all_to_all():
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29741", os.path.join(ROOT, "tests", "mp_moe_worker.py")]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=400, env=env, cwd=ROOT)
    assert out.returncode == 0, "\n".join(l for l in out.stderr.splitlines() if l.startswith("[rank0]"))[-4000:]
    res = json.loads([l for l in out.stdout.splitlines() if l.startswith("RESULT ")][-1][len("RESULT "):])
    assert max(res.values()) < 2e-2


def test_muon_gathers_tp_shards_over_peer_memory():
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29745", os.path.join(ROOT, "tests", "mp_muon_gather_worker.py")]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=env, cwd=ROOT)
    assert out.returncode == 0, "\n".join(l for l in out.stderr.splitlines() if l.startswith("[rank0]"))[-4000:]
    res = json.loads([l for l in out.stdout.splitlines() if l.startswith("RESULT ")][-1][len("RESULT "):])
    assert res == {"rows": True, "cols": True, "blocks": True}     # every case took the peer path


def test_context_parallel_attention_over_peer_memory_matches_packed_keys_and_fp32():
    """CP=2: K / V gathered over peer memory and addressed by global position inside the attention kernels, against
    the packed-keys path over NCCL and fp32 attention over the whole sequence (forward, dq, dk, dv)."""
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29751", os.path.join(ROOT, "tests", "mp_cp_attention_worker.py")]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=env, cwd=ROOT)
    assert out.returncode == 0, "\n".join(l for l in out.stderr.splitlines() if l.startswith("[rank0]"))[-4000:]
    res = json.loads([l for l in out.stdout.splitlines() if l.startswith("RESULT ")][-1][len("RESULT "):])
    assert res["worst_over_ranks"] < 2e-2, res
