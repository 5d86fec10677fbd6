"""One inference replica per node: launch the vLLM server, announce it, take it down again.

What the rest of the system observes (and what the reference's controller,
``steptronoss/generation/vllm/vllm_controller.py:19-143``, shares with this one):

* the server command comes from ``cfg.get_entrypoint_command_and_envs()`` and runs with ``PORT_SERVING`` set to a
  free port and ``VLLM_SERVER_DEV_MODE=1`` (the weight-reload RPCs only exist in dev mode);
* the replica counts as up when ``GET /health`` on that port answers 200;
* it is announced in the experiment store (``VLLM_NUM_WORKERS_OF_<model>`` = ``$NNODES``, its ``ip:port`` appended
  to the list ``VLLM_WORKERS_OF_<model>``) and to the router found under ``VLLM_ROUTER_ADDR_PORT_<key>``
  (``GET /register?endpoint=ip:port``), and withdrawn with ``GET /unregister`` when the controller stops;
* the server runs in its own process group, so stopping the controller stops the engine's children too.
"""
from __future__ import annotations

import atexit
import os
import signal
import subprocess
import sys
import time

from ...utils.general import get_free_port, get_my_ip
from ...utils.logger import logger

HEALTHY_CHECK_INTERVAL = 10


class _ServerProcess:
    """The server as a child process that leads its own process group."""

    def __init__(self, command: str, env: dict):
        self.popen = subprocess.Popen(command, shell=True, env={**os.environ, **env}, stdout=sys.stdout,  # noqa: S602
                                      stderr=sys.stderr, start_new_session=True)

    def exited(self) -> bool:
        return self.popen.poll() is not None

    def stop(self, grace_s: float = 5.0) -> None:
        if self.exited():
            return
        os.killpg(self.popen.pid, signal.SIGTERM)
        try:
            self.popen.wait(timeout=grace_s)
        except subprocess.TimeoutExpired:
            logger.warning(f"inference server (pid {self.popen.pid}) ignored SIGTERM for {grace_s:.0f} s: killing its group")
            os.killpg(self.popen.pid, signal.SIGKILL)
            self.popen.wait()


def _router_call(base_url: str, route: str, endpoint: str) -> bool:
    """``GET <router>/<route>?endpoint=...``; the router being away is reported, not raised."""
    import requests

    try:
        answer = requests.get(f"{base_url}/{route}", params={"endpoint": endpoint}, timeout=5)
    except requests.exceptions.RequestException as exc:
        logger.warning(f"router {base_url} did not take /{route} of {endpoint}: {exc}")
        return False
    if answer.status_code != 200:
        logger.warning(f"router {base_url} answered {answer.status_code} to /{route} of {endpoint}: {answer.text}")
        return False
    return True


class VLLMController:
    def __init__(self, cfg, health_interval: float = HEALTHY_CHECK_INTERVAL):
        self.cfg = cfg
        self.health_interval = health_interval
        self.nnodes = int(os.environ.get("NNODES", "1"))   # how many replicas the clients should expect
        self.vllm_port: int | None = None
        self.endpoint: str | None = None
        self.router_url: str | None = None
        self._server: _ServerProcess | None = None
        self._stopped = False

    @property
    def process(self):
        """The server's ``Popen`` (``None`` before ``run_vllm``)."""
        return None if self._server is None else self._server.popen

    # ------------------------------------------------------------------ the sequence `start` runs
    def start(self) -> None:
        """Launch, wait, announce, then stay with the server until it exits."""
        signal.signal(signal.SIGTERM, self._on_sigterm)
        atexit.register(self.shutdown)
        self.run_vllm()
        self.wait_for_health()
        self.register()
        self._server.popen.wait()

    def command_and_env(self) -> tuple[str, dict]:
        command, env = self.cfg.get_entrypoint_command_and_envs()
        self.vllm_port = get_free_port()
        return command, {**env, "PORT_SERVING": str(self.vllm_port), "VLLM_SERVER_DEV_MODE": "1"}

    def run_vllm(self) -> None:
        command, env = self.command_and_env()
        logger.info(f"starting the inference server on port {self.vllm_port}: {command}")
        self._server = _ServerProcess(command, env)

    def wait_for_health(self) -> None:
        import requests

        probe = f"http://localhost:{self.vllm_port}/health"
        waited = 0.0
        while True:
            time.sleep(self.health_interval)
            waited += self.health_interval
            if self._server is not None and self._server.exited():
                raise RuntimeError(f"the inference server exited with code {self._server.popen.returncode} before it "
                                   f"became healthy")
            try:
                if requests.get(probe, timeout=5).status_code == 200:
                    logger.info(f"inference server healthy after {waited:.0f} s")
                    return
            except requests.exceptions.RequestException:
                pass                                   # not listening yet
            logger.info(f"inference server not healthy yet ({waited:.0f} s)")

    def register(self) -> None:
        from ...utils.comm_utils import block_get_redis, get_exp_redis

        store = get_exp_redis()
        router = block_get_redis(store, f"VLLM_ROUTER_ADDR_PORT_{self.cfg.router_addr_key}")
        self.router_url = "http://" + (router.decode() if isinstance(router, bytes) else str(router))
        self.endpoint = f"{get_my_ip()}:{self.vllm_port}"
        model = self.cfg.model_name
        store.set(f"VLLM_NUM_WORKERS_OF_{model}", self.nnodes)
        store.rpush(f"VLLM_WORKERS_OF_{model}", self.endpoint)
        if _router_call(self.router_url, "register", self.endpoint):
            logger.info(f"replica {self.endpoint} announced to {self.router_url}")

    def deregister(self) -> None:
        if self.router_url and self.endpoint:
            _router_call(self.router_url, "unregister", self.endpoint)

    # ------------------------------------------------------------------ stopping
    def shutdown(self) -> None:
        """Withdraw the replica from the router and stop the server; safe to call more than once."""
        if self._stopped:
            return
        self._stopped = True
        self.deregister()
        if self._server is not None:
            self._server.stop()

    def _on_sigterm(self, signum, frame):
        self.shutdown()
        raise SystemExit(0)
