"""Per-node controller of one vLLM server: start it, wait until it answers, register it with the router,
deregister and stop it on exit (reference ``steptronoss/generation/vllm/vllm_controller.py:19-143``)."""
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


class VLLMController:
    def __init__(self, cfg, health_interval: float = HEALTHY_CHECK_INTERVAL):
        self.cfg = cfg
        self.process: subprocess.Popen | None = None
        self.vllm_port: int | None = None
        self.endpoint: str | None = None
        self.router_url: str | None = None
        self.health_interval = health_interval
        self._shutdown_called = False
        self.nnodes = int(os.environ.get("NNODES", "1"))  # replicas the clients should wait for

    def start(self):
        signal.signal(signal.SIGTERM, self._handle_sigterm)
        atexit.register(self.shutdown)
        self.run_vllm()
        self.wait_for_health()
        self.register()
        self.process.wait()

    def command_and_env(self) -> tuple[str, dict]:
        cmd, env = self.cfg.get_entrypoint_command_and_envs()
        self.vllm_port = get_free_port()
        env = dict(env, PORT_SERVING=str(self.vllm_port), VLLM_SERVER_DEV_MODE="1")  # reload RPCs need dev mode
        return cmd, env

    def run_vllm(self):
        cmd, env = self.command_and_env()
        logger.info(f"Launching vLLM with command: {cmd}")
        self.process = subprocess.Popen(cmd, shell=True, env=os.environ | env, stdout=sys.stdout,  # noqa: S602
                                        stderr=sys.stderr, preexec_fn=os.setsid)

    def wait_for_health(self):
        import requests

        url = f"http://localhost:{self.vllm_port}/health"
        logger.info("Waiting for health check to pass...")
        while True:
            time.sleep(self.health_interval)
            if self.process is not None and self.process.poll() is not None:
                raise RuntimeError("VLLM process dead.")
            try:
                if requests.get(url, timeout=5).status_code == 200:
                    return
            except requests.exceptions.RequestException as e:
                logger.info(f"Health check request failed: {e}, continue waiting...")

    def register(self):
        import requests

        from ...utils.comm_utils import block_get_redis, get_exp_redis

        store = get_exp_redis()
        router = block_get_redis(store, f"VLLM_ROUTER_ADDR_PORT_{self.cfg.router_addr_key}").decode()
        self.router_url = f"http://{router}"
        self.endpoint = f"{get_my_ip()}:{self.vllm_port}"
        name = self.cfg.model_name
        store.set(f"VLLM_NUM_WORKERS_OF_{name}", self.nnodes)
        store.rpush(f"VLLM_WORKERS_OF_{name}", self.endpoint)
        try:
            r = requests.get(f"{self.router_url}/register", params={"endpoint": self.endpoint}, timeout=5)
            if r.status_code == 200:
                logger.info(f"Registered endpoint {self.endpoint} to router {self.router_url}.")
            else:
                logger.warning(f"Router register failed: {r.status_code} {r.text}")
        except requests.exceptions.RequestException as exc:
            logger.warning(f"Router register request failed: {exc}")

    def deregister(self):
        import requests

        if not self.router_url or not self.endpoint:
            return
        try:
            requests.get(f"{self.router_url}/unregister", params={"endpoint": self.endpoint}, timeout=5)
        except requests.exceptions.RequestException as exc:
            logger.warning(f"Router unregister request failed: {exc}")

    def shutdown(self):
        if self._shutdown_called:
            return
        self._shutdown_called = True
        self.deregister()
        self._terminate()

    def _terminate(self):
        if self.process is None or self.process.poll() is not None:
            return
        try:
            os.killpg(self.process.pid, signal.SIGTERM)  # the server's own process group, started with setsid
            self.process.wait(timeout=5)
        except subprocess.TimeoutExpired:
            logger.warning("vLLM did not exit in time; force killing.")
            os.killpg(self.process.pid, signal.SIGKILL)

    def _handle_sigterm(self, signum, frame):
        self.shutdown()
        raise SystemExit(0)
