"""``torchrun`` with its multi-node arguments filled in from a rendezvous in the experiment store.

Every node runs ``NNODES=<n> EXP_ID=<id> python -m steptronoss_b200.launch.smartrun exp.py ...``; the nodes
append their address to one list in the store, the first entry becomes the master, the position in the list
the node rank.  One process per visible GPU (one process on a CPU node).
"""
from __future__ import annotations

import os
import socket
import subprocess
import sys
import time


def rendezvous(num_nodes: int, exp_id: str, poll_s: float = 1.0, store=None) -> tuple[int, str]:
    """``(node_rank, master_addr)`` once ``num_nodes`` nodes have checked in."""
    if num_nodes <= 1:
        return 0, "127.0.0.1"
    from ..utils.comm_utils import get_exp_redis

    store = store or get_exp_redis()
    key = f"SMARTRUN_RDZVS_{exp_id.replace('/', '_')}"
    try:
        me = socket.gethostbyname(socket.getfqdn(socket.gethostname()))
    except OSError:
        me = "127.0.0.1"
    me = f"{me}#{os.getpid()}" if os.environ.get("SMARTRUN_UNIQUE_PER_PROCESS") else me
    store.rpush(key, me)
    while True:
        addrs = [a.decode() for a in store.lrange(key)]
        if len(addrs) >= num_nodes:
            break
        if addrs and addrs[0] == me:
            print(f"\033[33m{len(addrs)} / {num_nodes} Nodes Ready.\033[0m", flush=True)
        time.sleep(poll_s)
    rank = addrs.index(me)
    if rank == 0:
        store.expire(key, 60)
    return rank, addrs[0].split("#")[0]


def torchrun_command(argv: list, num_nodes: int, node_rank: int, master_addr: str, master_port: int,
                     nproc: int) -> list:
    return [sys.executable, "-m", "torch.distributed.run", "--nnodes", str(num_nodes), "--nproc-per-node", str(nproc),
            "--node-rank", str(node_rank), "--master-addr", master_addr, "--master-port", str(master_port), *argv]


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    import torch

    nproc = max(torch.cuda.device_count(), 1)
    num_nodes = int(os.environ.get("NNODES", "1"))
    exp_id = os.environ.get("EXP_ID", "local")
    rank, master = rendezvous(num_nodes, exp_id)
    cmd = torchrun_command(argv, num_nodes, rank, master, int(os.environ.get("MASTER_PORT", 12345)), nproc)
    print("Modified Command:\n\033[32m" + " ".join(cmd) + "\033[0m", flush=True)
    return subprocess.call(cmd)


if __name__ == "__main__":
    sys.exit(main())
