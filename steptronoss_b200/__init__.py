"""steptronoss_b200: a B200-native LLM training framework with the SteptronOss surface."""
from __future__ import annotations

__version__ = "0.1.0"


def debug(rank: int | list = 0, stop: bool = False, any_rank: bool = False, base_port: int = 5000):
    """Wait for a remote debugger (``debugpy``, e.g. VS Code "attach") on the chosen ranks
    (reference ``steptronoss/__init__.py:1-72``).

    ``rank``: one rank or a list; the i-th listed rank listens on ``base_port + i`` (``any_rank``: every rank, on
    ``base_port + its rank``).  The call prints ``ip / port / rank``, blocks until a client connects, and with
    ``stop=True`` breaks right after.  Other ranks return at once; so does a process that already has a client.
    Returns the ``(host, port)`` it listened on, or ``None``."""
    import socket

    try:
        import debugpy
    except ImportError as e:  # a development dependency
        raise ImportError("steptronoss_b200.debug() needs the debugpy package") from e
    import torch.distributed as dist

    ranks = list(rank) if isinstance(rank, (list, tuple)) else [rank]
    if debugpy.is_client_connected():
        return None
    me = dist.get_rank() if dist.is_available() and dist.is_initialized() else 0
    if not (any_rank or me in ranks):
        return None
    try:
        host = socket.gethostbyname(socket.getfqdn(socket.gethostname()))
    except OSError:
        host = "127.0.0.1"
    port = base_port + (me if any_rank else ranks.index(me))
    debugpy.listen((host, port), in_process_debug_adapter=False)
    print(f"waiting for a debugger: ip {host} port {port} rank {me}\a", flush=True)
    debugpy.wait_for_client()
    print("debugger connected", flush=True)
    if stop:
        debugpy.breakpoint()
    return host, port
