"""Round-robin HTTP front of the experiment's inference replicas.

Reference: ``steptronoss/generation/vllm/vllm_router.py:17-233``.  Replicas register themselves
(``GET /register?endpoint=host:port``), clients post OpenAI-style requests to ``/v1/<route>`` and the router
forwards each to the next replica, streaming the answer back when the request asks for it.  The router
publishes its own address in the experiment store under ``VLLM_ROUTER_ADDR_PORT_<router_addr_key>``.
"""
from __future__ import annotations

import json
import threading

from ...config import Config
from ...utils.general import get_free_port, get_my_ip

_DROP_REQ = {"host", "content-length"}
_DROP_RESP = {"content-length", "transfer-encoding", "connection"}


class VLLMRouterConfig(Config):
    router_addr_key: str = "default"
    routed_methods: dict = {"completions": ["POST"], "chat/completions": ["POST"]}

    def run(self):
        VLLMRouter(cfg=self).serve()


class VLLMRouter:
    def __init__(self, cfg: VLLMRouterConfig):
        from fastapi import FastAPI

        self.cfg = cfg
        self._endpoints: list = []
        self._lock = threading.Lock()
        self._rr = 0
        self._session = None
        app = FastAPI()
        app.add_api_route("/register", self.register, methods=["GET"])
        app.add_api_route("/unregister", self.unregister, methods=["GET"])
        app.add_api_route("/get_info", self.get_info, methods=["GET"])
        for route, methods in cfg.routed_methods.items():
            app.add_api_route(f"/v1/{route}", self._make_proxy(route), methods=list(methods))
        self.app = app

    # ------------------------------------------------------------------ registry
    def register(self, endpoint: str) -> bool:
        with self._lock:
            if endpoint in self._endpoints:
                return False
            self._endpoints.append(endpoint)
            return True

    def unregister(self, endpoint: str) -> bool:
        with self._lock:
            if endpoint not in self._endpoints:
                return False
            self._endpoints.remove(endpoint)
            return True

    def get_info(self) -> list:
        with self._lock:
            return [{"endpoint": e} for e in self._endpoints]

    def select_endpoint(self) -> str:
        from fastapi import HTTPException

        with self._lock:
            if not self._endpoints:
                raise HTTPException(status_code=503, detail="No endpoints registered")
            e = self._endpoints[self._rr % len(self._endpoints)]
            self._rr = (self._rr + 1) % len(self._endpoints)
            return e

    # ------------------------------------------------------------------ serving
    def serve(self, port: int | None = None, publish: bool = True):
        import uvicorn

        port = port or get_free_port()
        if publish:
            from ...utils.comm_utils import get_exp_redis

            get_exp_redis().set(f"VLLM_ROUTER_ADDR_PORT_{self.cfg.router_addr_key}", f"{get_my_ip()}:{port}")
        uvicorn.run(self.app, host="0.0.0.0", port=port, access_log=False)

    async def _get_session(self):
        import aiohttp

        if self._session is None or self._session.closed:
            # no router-side timeout and no connection cap: the client decides, and the replicas batch
            self._session = aiohttp.ClientSession(
                connector=aiohttp.TCPConnector(limit=0, limit_per_host=0),
                timeout=aiohttp.ClientTimeout(total=None, connect=None, sock_connect=None, sock_read=None))
        return self._session

    @staticmethod
    def _url(endpoint: str) -> str:
        return endpoint if endpoint.startswith(("http://", "https://")) else f"http://{endpoint}"

    def _make_proxy(self, route: str):
        from fastapi import HTTPException, Request, Response
        from fastapi.responses import StreamingResponse

        async def proxy(request: Request):
            import aiohttp

            url = f"{self._url(self.select_endpoint())}/v1/{route}"
            params = dict(request.query_params)
            headers = {k: v for k, v in request.headers.items() if k.lower() not in _DROP_REQ}
            body = await request.body()
            try:
                session = await self._get_session()
                upstream = await session.request(request.method, url, params=params, data=body, headers=headers)
            except aiohttp.ClientError as exc:
                raise HTTPException(status_code=502, detail=str(exc)) from exc
            out_headers = {k: v for k, v in upstream.headers.items() if k.lower() not in _DROP_RESP}
            stream = params.get("stream") in {"1", "true", "True"}
            if not stream and body and "application/json" in request.headers.get("content-type", "").lower():
                try:
                    stream = json.loads(body).get("stream") is True
                except json.JSONDecodeError:
                    pass
            if "text/event-stream" in upstream.headers.get("content-type", "").lower():
                stream = True
            if stream:
                async def chunks():
                    try:
                        async for c in upstream.content.iter_any():
                            if c:
                                yield c
                    finally:
                        upstream.release()

                return StreamingResponse(chunks(), status_code=upstream.status, headers=out_headers,
                                         media_type=upstream.headers.get("content-type"))
            try:
                content = await upstream.read()
            finally:
                upstream.release()
            return Response(content=content, status_code=upstream.status, headers=out_headers)

        # annotations of this module are strings (postponed evaluation) and ``Request`` is a local name: hand
        # FastAPI the class itself, otherwise it takes ``request`` for a query parameter
        proxy.__annotations__ = {"request": Request}

        return proxy
