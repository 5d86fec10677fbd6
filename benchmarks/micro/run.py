"""Build and run the sm_100a micro-benchmarks behind the design of the attention kernels (one B200).

* ``sync_hop``         round trip between one issuing thread and 128 worker threads over two mbarriers
                       (``tcgen05.commit`` or a plain arrive one way, 128 arrives the other way);
* ``umma_rate``        cycles per ``tcgen05.mma`` step for the operand placements the kernels use (A in shared memory
                       or TMEM, B K-major or MN-major, N = 64 / 128 / 256), issued back to back by one thread, and the
                       same through the helpers of ``csrc/attention_common.cuh`` with a commit per tile;
* ``tmem_contention``  the Q K^T / P V chain of the forward kernel while four other warps load (and store) their TMEM
                       lanes in a loop: cycles per step of the chain and how many 128-column loads a warp completes.

    python benchmarks/micro/run.py            # all three
    python benchmarks/micro/run.py umma_rate
"""
from __future__ import annotations

import os
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(os.path.dirname(os.path.dirname(HERE)), "steptronoss_b200", "csrc")
NAMES = ("sync_hop", "umma_rate", "tmem_contention")


def main():
    names = sys.argv[1:] or NAMES
    nvcc = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    out_dir = tempfile.mkdtemp(prefix="stb200_micro_")
    for name in names:
        exe = os.path.join(out_dir, name)
        cmd = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-I", CSRC, "-o", exe,
               os.path.join(HERE, name + ".cu"), os.path.join(CSRC, "host_util.cu"), "-lcudart"]
        subprocess.run(cmd, check=True)
        print(f"== {name}", flush=True)
        subprocess.run([exe], check=True, timeout=120)


if __name__ == "__main__":
    main()
