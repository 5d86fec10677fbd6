"""Client of the experiment's inference service (reference ``steptronoss/generation/vllm/vllm_client.py:18-195``):
finds the router through the experiment store, waits for the expected number of replicas, sends completions and
makes every replica reload weights from a directory."""
from __future__ import annotations

import asyncio
import time
from functools import cached_property
from typing import Any

from ...utils.general import retry_on, run_async
from ...utils.logger import logger

ROUTER_ADDR_KEY = "VLLM_ROUTER_ADDR_PORT"


class VLLMClient:
    def __init__(self, cfg):
        import requests

        self.cfg = cfg
        self.session = requests.Session()
        self.session.proxies = {"http": ""}
        self.asession = None

    def close(self) -> None:
        if self.asession is not None:
            try:
                run_async(self.asession.close())
            finally:
                self.asession = None
        if self.session is not None:
            self.session.close()
            self.session = None

    async def aclose(self) -> None:
        if self.asession is not None:
            try:
                await self.asession.close()
            finally:
                self.asession = None
        if self.session is not None:
            self.session.close()
            self.session = None

    @retry_on((ConnectionError, IOError), retries=3)
    def post(self, url: str, **kw):
        return self.session.post(url, **kw).json()

    @retry_on((ConnectionError, IOError), retries=3)
    def get(self, url: str, params: dict | None = None):
        return self.session.get(url, params=params or {}).json()

    async def _asession(self):
        import aiohttp

        if self.asession is None:
            self.asession = aiohttp.ClientSession(timeout=aiohttp.ClientTimeout(total=600, connect=60, sock_read=600))
        return self.asession

    async def apost(self, url: str, decode_json: bool = True, **kw):
        s = await self._asession()
        async with s.post(url, **kw) as r:
            return await (r.json() if decode_json else r.read())

    async def aget(self, url: str, params: dict | None = None):
        s = await self._asession()
        async with s.get(url, params=params or {}) as r:
            return await r.json()

    @cached_property
    def _router_addr(self) -> str:
        from ...utils.comm_utils import block_get_redis, get_exp_redis

        key = f"{ROUTER_ADDR_KEY}_{self.cfg.router_addr_key}"
        return f"http://{block_get_redis(get_exp_redis(), key).decode()}"

    def check_server_alive(self) -> bool:
        try:
            out = self.post(f"{self._router_addr}/v1/completions", headers={"Content-Type": "application/json"},
                            json={"model": self.cfg.model_name, "prompt": "ping", "max_tokens": 3})
            return bool(out["choices"][0])
        except Exception:
            return False

    def wait_for_server(self, timeout: int = 3600) -> list:
        """Block until the expected number of replicas is registered and answering; return their endpoints."""
        from ...utils.comm_utils import block_get_redis, get_exp_redis

        expected = int(block_get_redis(get_exp_redis(), f"VLLM_NUM_WORKERS_OF_{self.cfg.model_name}", timeout=timeout))
        t0 = time.time()
        while time.time() - t0 < timeout:
            eps = [e["endpoint"] for e in self.get(f"{self._router_addr}/get_info")]
            logger.info(f"[wait_for_server] {len(eps)}/{expected} endpoints ready: {eps}")
            if len(eps) >= expected and self.check_server_alive():
                assert len(eps) == len(set(eps)), "Duplicate endpoints found"
                return eps
            time.sleep(max(2, timeout / 1200))
        raise TimeoutError("VLLM wait server timeout!")

    def completion(self, prompt_or_request: Any, max_tokens: int | None = None) -> dict:
        if hasattr(prompt_or_request, "model_dump"):
            payload = prompt_or_request.model_dump()
        elif isinstance(prompt_or_request, dict):
            payload = dict(prompt_or_request)
        else:
            payload = {"prompt": prompt_or_request, "return_token_ids": True}
        payload["model"] = self.cfg.model_name
        if max_tokens:
            payload["max_tokens"] = max_tokens
        return self.post(f"{self._router_addr}/v1/completions", json=payload)

    async def _reload_endpoint(self, endpoint: str, new_path: str | None) -> bool:
        await self.apost(f"http://{endpoint}/collective_rpc",
                         json={"method": "reload_weights", "kwargs": {"weights_path": new_path} if new_path else {}})
        await self.apost(f"http://{endpoint}/reset_prefix_cache", decode_json=False)
        return True

    def reload_weights(self, new_path: str | None = None) -> bool:
        endpoints = self.wait_for_server()

        async def run():
            try:
                return all(await asyncio.gather(*[self._reload_endpoint(e, new_path) for e in endpoints]))
            finally:
                if self.asession is not None:
                    await self.asession.close()
                    self.asession = None

        return run_async(run())
