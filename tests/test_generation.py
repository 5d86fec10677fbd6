"""Generation side-car: in-process and multi-process generation controllers, the round-robin router in front of
fake replicas, and the per-node server controller with a fake server process."""
import json
import threading
import time
from http.server import BaseHTTPRequestHandler, HTTPServer

import pytest

from tests.gen_items import Rollout, Square


def test_single_controller_runs_items_and_reports_errors():
    from steptronoss_b200.generation.async_generation import SingleGenerationController

    c = SingleGenerationController()
    try:
        got = {item.x: res for item, res in c.generate([Square(2), Square(3), Square(-1)])}
        assert got[2] == 4 and got[3] == 9 and isinstance(got[-1], RuntimeError) and "negative" in str(got[-1])
        tr = dict((item.x, res) for item, res in c.generate([Rollout(5)], for_train=True))
        assert tr[5] == [5, 6]
        bad = list(c.generate([Square(1)], for_train=True))          # not a TrainableItem
        assert isinstance(bad[0][1], RuntimeError)
    finally:
        c.shutdown()


def test_multi_process_controller_caps_items_in_flight():
    from steptronoss_b200.generation.async_generation import GenerationController

    c = GenerationController(num_workers=2, max_concurrent_genables=2, start_method="spawn")
    try:
        seen_inflight = []
        done = []
        lock = threading.Lock()

        def cb(item, res):
            with lock:
                done.append((item.x, res))

        c.set_tqdm(disabled=False, total=6, desc="squares")
        with pytest.raises(ValueError):
            c.set_tqdm(False, -1, "x")
        for i in range(6):
            c.submit_with_callback(Square(i, delay=0.15), callback=cb)
            seen_inflight.append(c.inflight_count)
        deadline = time.time() + 60
        while len(done) < 6 and time.time() < deadline:
            seen_inflight.append(c.inflight_count)
            time.sleep(0.02)
        assert sorted(done) == [(i, i * i) for i in range(6)]
        deadline = time.time() + 10
        while c.completed_count < 6 and time.time() < deadline:       # the count follows the callback
            time.sleep(0.01)
        assert max(seen_inflight) <= 2 and c.completed_count == 6
        assert c._bar is not None and c._bar.n == 6 and c._bar.total == 6 and c._bar.desc.startswith("squares")
        c.set_tqdm(disabled=True, total=0, desc="off")
        assert c._bar is None
        with pytest.raises(ValueError):
            GenerationController(num_workers=1, max_concurrent_genables=0)
    finally:
        c.shutdown()


class _Replica(BaseHTTPRequestHandler):
    def do_POST(self):  # noqa: N802
        n = int(self.headers.get("content-length", 0))
        body = json.loads(self.rfile.read(n) or b"{}")
        if body.get("stream"):
            self.send_response(200)
            self.send_header("content-type", "text/event-stream")
            self.end_headers()
            for i in range(3):
                self.wfile.write(f"data: {self.server.tag}-{i}\n\n".encode())
                self.wfile.flush()
            return
        out = json.dumps({"replica": self.server.tag, "echo": body.get("prompt"), "path": self.path}).encode()
        self.send_response(200)
        self.send_header("content-type", "application/json")
        self.send_header("content-length", str(len(out)))
        self.end_headers()
        self.wfile.write(out)

    def log_message(self, *a):
        pass


def _replica(tag):
    srv = HTTPServer(("127.0.0.1", 0), _Replica)
    srv.tag = tag
    threading.Thread(target=srv.serve_forever, daemon=True).start()
    return srv


def test_router_registers_and_forwards_round_robin():
    from fastapi.testclient import TestClient

    from steptronoss_b200.generation.vllm.vllm_router import VLLMRouter, VLLMRouterConfig

    router = VLLMRouter(VLLMRouterConfig())
    a, b = _replica("a"), _replica("b")
    try:
        with TestClient(router.app) as client:
            assert client.post("/v1/completions", json={"prompt": "x"}).status_code == 503     # nobody registered
            ea, eb = f"127.0.0.1:{a.server_port}", f"127.0.0.1:{b.server_port}"
            assert client.get("/register", params={"endpoint": ea}).json() is True
            assert client.get("/register", params={"endpoint": ea}).json() is False            # already known
            assert client.get("/register", params={"endpoint": eb}).json() is True
            assert [e["endpoint"] for e in client.get("/get_info").json()] == [ea, eb]
            tags = [client.post("/v1/completions", json={"prompt": f"p{i}"}).json() for i in range(4)]
            assert [t["replica"] for t in tags] == ["a", "b", "a", "b"]
            assert tags[0]["echo"] == "p0" and tags[0]["path"] == "/v1/completions"
            r = client.post("/v1/chat/completions", json={"prompt": "s", "stream": True})
            assert r.status_code == 200 and r.text.count("data: ") == 3
            assert client.get("/unregister", params={"endpoint": ea}).json() is True
            assert client.get("/unregister", params={"endpoint": ea}).json() is False
            assert {client.post("/v1/completions", json={}).json()["replica"] for _ in range(3)} == {"b"}
    finally:
        a.shutdown()
        b.shutdown()


def test_router_answers_502_when_a_replica_is_gone():
    from fastapi.testclient import TestClient

    from steptronoss_b200.generation.vllm.vllm_router import VLLMRouter, VLLMRouterConfig

    router = VLLMRouter(VLLMRouterConfig())
    dead = _replica("dead")
    port = dead.server_port
    dead.shutdown()
    dead.server_close()
    with TestClient(router.app) as client:
        client.get("/register", params={"endpoint": f"127.0.0.1:{port}"})
        assert client.post("/v1/completions", json={"prompt": "x"}).status_code == 502


class _FakeStore(dict):
    def set(self, k, v):
        self[k] = str(v).encode()

    def get(self, k):
        return dict.get(self, k)

    def rpush(self, k, v):
        self.setdefault(k, []).append(v)


def test_controller_starts_waits_registers_and_stops(monkeypatch):
    import sys

    import steptronoss_b200.utils.comm_utils as cu
    from steptronoss_b200.generation.vllm import vllm_controller as vc

    class Cfg:
        router_addr_key, model_name = "k", "m-e1"

        def get_entrypoint_command_and_envs(self):
            # the "server": an HTTP process that answers /health on $PORT_SERVING
            code = ("import os,http.server as h;"
                    "H=type('H',(h.BaseHTTPRequestHandler,),{'do_GET':lambda s:(s.send_response(200),s.end_headers()),"
                    "'log_message':lambda *a:None});"
                    "h.HTTPServer(('127.0.0.1',int(os.environ['PORT_SERVING'])),H).serve_forever()")
            return f'{sys.executable} -c "{code}"', {"EXTRA": "1"}

    calls = []

    class _Resp:
        status_code, text = 200, "true"

    store = _FakeStore()
    store.set("VLLM_ROUTER_ADDR_PORT_k", "127.0.0.1:1")
    monkeypatch.setattr(cu, "get_exp_redis", lambda: store)
    monkeypatch.setattr(cu, "block_get_redis", lambda s, k: s.get(k))
    import requests

    real_get = requests.get

    def fake_get(url, **kw):
        if url.startswith("http://127.0.0.1:1/"):
            calls.append((url.rsplit("/", 1)[1], kw["params"]["endpoint"]))
            return _Resp()
        return real_get(url, **kw)

    monkeypatch.setattr(requests, "get", fake_get)
    monkeypatch.setenv("NNODES", "3")
    c = vc.VLLMController(Cfg(), health_interval=0.2)
    cmd, env = c.command_and_env()
    assert env["VLLM_SERVER_DEV_MODE"] == "1" and env["EXTRA"] == "1" and env["PORT_SERVING"] == str(c.vllm_port)
    c.run_vllm()
    try:
        c.wait_for_health()
        c.register()
        assert calls == [("register", c.endpoint)] and c.endpoint.endswith(f":{c.vllm_port}")
        assert store["VLLM_NUM_WORKERS_OF_m-e1"] == b"3" and store["VLLM_WORKERS_OF_m-e1"] == [c.endpoint]
    finally:
        c.shutdown()
    assert calls[-1] == ("unregister", c.endpoint)
    assert c.process.poll() is not None
    c.shutdown()                                                        # idempotent
    assert [x[0] for x in calls].count("unregister") == 1


def test_deploy_command_lists_the_configured_options(monkeypatch):
    from steptronoss_b200.exp.inference import VLLMDeployConfig

    monkeypatch.setenv("EXP_ID", "run7/trainer")
    c = VLLMDeployConfig()
    c.model_config_path, c.max_seq_len, c.vllm_tp, c.vllm_dp, c.max_cache_size = "/m/q", 4096, 2, 4, 32
    c.reasoning_parser, c.enable_expert_parallel, c.vllm_enable_prefix_caching = "deepseek_r1", True, False
    c.vllm_hf_overrides = {"rope_scaling": None}
    c.vllm_mtp_num_tokens, c.vllm_mtp_method = 2, "mtp"
    c.load_weight_from_config_path = False
    cmd, env = c.get_entrypoint_command_and_envs()
    assert cmd.startswith("vllm serve /m/q --port $PORT_SERVING")
    for piece in ("--max-model-len 4096", "--tensor-parallel-size 2", "--data-parallel-size 4", "--max-num-seqs 32",
                  "--reasoning-parser deepseek_r1", "--enable-expert-parallel", "--no-enable-prefix-caching",
                  "--hf-overrides $HF_OVERRIDES", "--speculative-config $SPECULATIVE_CONFIG", "--load-format dummy",
                  "--tokenizer /m/q", "--trust-remote-code", "--enable-chunked-prefill"):
        assert piece in cmd, piece
    assert "--pipeline-parallel-size" not in cmd and "--enforce-eager" not in cmd
    assert json.loads(env["HF_OVERRIDES"].strip("'")) == {"rope_scaling": None}
    assert json.loads(env["SPECULATIVE_CONFIG"].strip("'")) == {"num_speculative_tokens": 2, "method": "mtp"}
    assert "run7" in c.model_name and f"--served-model-name {c.model_name}" in cmd


class _Server(BaseHTTPRequestHandler):
    """Plays the router (/get_info, /v1/completions) and a replica (/collective_rpc, /reset_prefix_cache)."""

    def _send(self, obj):
        out = json.dumps(obj).encode()
        self.send_response(200)
        self.send_header("content-type", "application/json")
        self.send_header("content-length", str(len(out)))
        self.end_headers()
        self.wfile.write(out)

    def do_GET(self):  # noqa: N802
        self.server.log.append(("GET", self.path))
        self._send([{"endpoint": f"127.0.0.1:{self.server.server_port}"}])

    def do_POST(self):  # noqa: N802
        n = int(self.headers.get("content-length", 0))
        body = json.loads(self.rfile.read(n) or b"{}")
        self.server.log.append(("POST", self.path, body))
        self._send({"choices": [{"text": "pong", "token_ids": [1]}]} if "completions" in self.path else {"ok": True})

    def log_message(self, *a):
        pass


def test_client_waits_completes_and_reloads_weights(monkeypatch):
    import steptronoss_b200.utils.comm_utils as cu
    from steptronoss_b200.generation.vllm.vllm_client import VLLMClient

    srv = HTTPServer(("127.0.0.1", 0), _Server)
    srv.log = []
    threading.Thread(target=srv.serve_forever, daemon=True).start()

    class Cfg:
        router_addr_key, model_name = "k", "m"

    store = _FakeStore()
    store.set("VLLM_ROUTER_ADDR_PORT_k", f"127.0.0.1:{srv.server_port}")
    store.set("VLLM_NUM_WORKERS_OF_m", 1)
    monkeypatch.setattr(cu, "get_exp_redis", lambda: store)
    monkeypatch.setattr(cu, "block_get_redis", lambda s, k, timeout=None: s.get(k))
    cli = VLLMClient(Cfg())
    try:
        assert cli.wait_for_server(timeout=20) == [f"127.0.0.1:{srv.server_port}"]
        out = cli.completion("hello", max_tokens=5)
        assert out["choices"][0]["text"] == "pong"
        sent = [x for x in srv.log if x[0] == "POST" and x[1] == "/v1/completions"][-1][2]
        assert sent == {"prompt": "hello", "return_token_ids": True, "model": "m", "max_tokens": 5}
        assert cli.reload_weights("/hot") is True
        rpc = [x for x in srv.log if x[0] == "POST" and x[1] == "/collective_rpc"][-1][2]
        assert rpc == {"method": "reload_weights", "kwargs": {"weights_path": "/hot"}}
        assert any(x[1] == "/reset_prefix_cache" for x in srv.log)
    finally:
        cli.close()
        srv.shutdown()


def test_deploy_training_model_writes_hf_weights_and_asks_the_servers_to_reload(tmp_path, monkeypatch):
    """Weight push of an RL step: the training model goes to ``hot_path`` as safetensors in HF naming, then the
    servers are told to load that directory."""
    import json

    import torch

    from steptronoss_b200.exp.inference import VLLMDeployConfig
    from steptronoss_b200.models.qwen_dense import QwenModel
    from steptronoss_b200.parallel.state import PM
    from tests.tiny_exp import make_tiny_exp

    PM.initialize()
    exp = make_tiny_exp(gbs=1, seq=32, iters=1, layers=1, hidden=32, heads=4, kv_heads=2, head_dim=8, ffn=64, vocab=64)
    PM.set_mesh(exp.model_cfg.parallel_cfg)
    model = QwenModel(cfg=exp.model_cfg, layer_map=exp.model_cfg.build_layer_map())
    model.init_weights(0, 0.02)
    calls = []

    class FakeClient:
        def wait_for_server(self):
            calls.append("wait")

        def reload_weights(self, path):
            calls.append(("reload", path))

    cfg = VLLMDeployConfig()
    cfg.hot_path = str(tmp_path / "hot")
    cfg.model_config_path = ""
    monkeypatch.setattr(type(cfg), "build_cli", lambda self: FakeClient())
    cfg.deploy_training_model([model])
    assert calls == ["wait", ("reload", str(tmp_path / "hot")), "wait"]
    index = json.load(open(tmp_path / "hot" / "model.safetensors.index.json"))
    names = set(index["weight_map"])
    assert "model.embed_tokens.weight" in names and "model.layers.0.self_attn.q_proj.weight" in names
    from safetensors.torch import load_file

    shard = load_file(str(tmp_path / "hot" / sorted(set(index["weight_map"].values()))[0]))
    assert torch.equal(shard["model.embed_tokens.weight"], model.tok_embeddings.word_embeddings.weight.detach())
