"""Experiment-wide rendezvous and work queues.

The processes of one experiment (trainer ranks, generation workers, the request router, evaluation workers)
share one small key/value + list server, the *experiment store* (``csrc/expstore/expstore_server.cpp``, a
single-threaded epoll server).  The first process that needs it elects itself on the shared file system and
starts the server; everyone else reads the address from the rendezvous file.

Reference: ``steptronoss/utils/comm_utils.py:33-670`` (which spawns a redis-server for the same purpose).
The election protocol is the reference's: directory ``STEPTRON_MEET_DIR``, file
``redis-rendezvous-<exp id>.pkl`` created with ``O_EXCL``, considered stale after 24 h, and
``CANNOT_BE_REDIS_SERVER=1`` keeps a process from becoming the host.
"""
from __future__ import annotations

import os
import pickle
import socket
import struct
import subprocess
import threading
import time
import uuid
from collections.abc import Iterable
from pathlib import Path
from queue import Empty

_OPS = dict(ping=0, set=1, get=2, delete=3, incr=4, lpush=5, rpush=6, lpop=7, rpop=8, llen=9, keys=10, setnx=11,
            expire=12, zadd=13, zincrby=14, zpopmin_incr=15, shutdown=16, lrange=17)
_SERVER_BIN = Path(__file__).resolve().parent.parent / "_native" / "stb_expstore"

STORE = None
IS_STORE_HOST = False
STORE_ADDR: str | None = None
STORE_PORT: int | None = None
_SERVER_PROC = None
_LOCK = threading.Lock()
_THREAD_LOCAL = threading.local()


def get_exp_id() -> str:
    return os.environ.get("EXP_ID", "local")


def _b(x) -> bytes:
    if isinstance(x, bytes):
        return x
    if isinstance(x, str):
        return x.encode()
    return str(x).encode()


class ExpStore:
    """Client of the experiment store (one TCP connection per thread).  The method names follow the redis
    client the reference uses, values are bytes."""

    def __init__(self, host: str, port: int, connect_timeout: float = 1200.0):
        self.host, self.port, self.connect_timeout = host, int(port), connect_timeout
        self._local = threading.local()

    def _sock(self):
        s = getattr(self._local, "sock", None)
        if s is None:
            deadline = time.monotonic() + self.connect_timeout
            while True:
                try:
                    s = socket.create_connection((self.host, self.port), timeout=30)
                    break
                except OSError:
                    if time.monotonic() > deadline:
                        raise
                    time.sleep(0.2)
            s.setsockopt(socket.IPPROTO_TCP, socket.TCP_NODELAY, 1)
            s.settimeout(1200)
            self._local.sock = s
        return s

    def _recv(self, s, n: int) -> bytes:
        buf = bytearray()
        while len(buf) < n:
            chunk = s.recv(n - len(buf))
            if not chunk:
                raise ConnectionError("experiment store closed the connection")
            buf += chunk
        return bytes(buf)

    def _call(self, op: str, key=b"", payload: bytes = b""):
        key = _b(key)
        body = struct.pack("<BI", _OPS[op], len(key)) + key + payload
        for attempt in range(3):
            try:
                s = self._sock()
                s.sendall(struct.pack("<I", len(body)) + body)
                (n,) = struct.unpack("<I", self._recv(s, 4))
                data = self._recv(s, n)
                break
            except (ConnectionError, OSError):
                self._local.sock = None
                if attempt == 2:
                    raise
                time.sleep(0.2 * (attempt + 1))
        status, out = data[0], data[1:]
        if status == 2:
            raise RuntimeError(f"experiment store: {out.decode(errors='replace')}")
        return None if status == 1 else out

    # strings / counters
    def ping(self) -> bool:
        return self._call("ping") == b"PONG"

    def set(self, key, value) -> None:
        self._call("set", key, _b(value))

    def setnx(self, key, value) -> bool:
        return self._call("setnx", key, _b(value)) is not None

    def get(self, key):
        return self._call("get", key)

    def delete(self, key) -> bool:
        return self._call("delete", key) is not None

    def incr(self, key, amount: int = 1) -> int:
        return struct.unpack("<q", self._call("incr", key, struct.pack("<q", amount)))[0]

    def decr(self, key, amount: int = 1) -> int:
        return self.incr(key, -amount)

    def expire(self, key, seconds: float) -> None:
        self._call("expire", key, struct.pack("<d", float(seconds)))

    def keys(self, pattern: str = "") -> list:
        out = self._call("keys", pattern.rstrip("*"))
        return [k for k in out.split(b"\n") if k]

    # lists
    def lpush(self, key, value) -> int:
        return struct.unpack("<q", self._call("lpush", key, _b(value)))[0]

    def rpush(self, key, value) -> int:
        return struct.unpack("<q", self._call("rpush", key, _b(value)))[0]

    def lpop(self, key):
        return self._call("lpop", key)

    def rpop(self, key):
        return self._call("rpop", key)

    def llen(self, key) -> int:
        return struct.unpack("<q", self._call("llen", key))[0]

    def lrange(self, key) -> list:
        raw, out, off = self._call("lrange", key), [], 0
        while off < len(raw):
            (n,) = struct.unpack_from("<I", raw, off)
            out.append(raw[off + 4: off + 4 + n])
            off += 4 + n
        return out

    def brpop(self, key, timeout: float | None = None, interval: float = 0.05):
        t0 = time.monotonic()
        while True:
            v = self.rpop(key)
            if v is not None:
                return v
            if timeout is not None and time.monotonic() - t0 > timeout:
                return None
            time.sleep(interval)

    # scored sets (sub-queue balancing)
    def zadd(self, key, mapping: dict) -> None:
        for member, score in mapping.items():
            self._call("zadd", key, struct.pack("<d", float(score)) + _b(member))

    def zincrby(self, key, amount: float, member) -> None:
        self._call("zincrby", key, struct.pack("<d", float(amount)) + _b(member))

    def zpopmin_incr(self, key):
        """The member with the lowest score, whose score is raised by one in the same step."""
        return self._call("zpopmin_incr", key)

    def shutdown(self) -> None:
        try:
            self._call("shutdown")
        except Exception:
            pass


def start_store_server(port: int = 0) -> tuple[subprocess.Popen, int]:
    """Start the server (building it when the binary is missing) and return ``(process, port)``."""
    if not _SERVER_BIN.exists():
        from ..csrc.build import build_expstore

        build_expstore()
    proc = subprocess.Popen([str(_SERVER_BIN), str(port)], stdout=subprocess.PIPE, text=True)
    line = proc.stdout.readline()
    if not line.startswith("EXPSTORE_PORT"):
        proc.kill()
        raise RuntimeError(f"experiment store did not start: {line!r}")
    return proc, int(line.split()[1])


def safely_start_redis(retries: int = 3, wait_per_retry: float = 1.0) -> int:
    """Start the store server on a free port, check that it answers (a write read back), and return the port; a
    failed start is retried.  The reference's name and return value for the same step (utils/comm_utils.py:33-100):
    the server process stays with this module, ``reset_exp_store`` stops it."""
    global _SERVER_PROC
    last = None
    for _ in range(max(1, retries)):
        try:
            proc, port = start_store_server()
            probe = ExpStore("127.0.0.1", port, connect_timeout=10)
            probe.set("redis_start_mark", str(os.getpid()))
            if probe.get("redis_start_mark") == str(os.getpid()).encode():
                probe.delete("redis_start_mark")
                _SERVER_PROC = proc
                return port
            proc.kill()
        except Exception as e:                  # a port taken between the pick and the bind, a slow start
            last = e
        time.sleep(wait_per_retry)
    raise RuntimeError(f"could not start the experiment store after {retries} attempts: {last}")


def block_get_redis(client: ExpStore, key: str, timeout: float = 1200, interval: float = 1.0):
    """Poll ``key`` until it exists (name kept from the reference)."""
    t0 = time.time()
    while True:
        v = client.get(key)
        if v is not None:
            return v
        if time.time() - t0 > timeout:
            raise TimeoutError(f"Timeout waiting for {key}")
        time.sleep(interval)


block_get = block_get_redis


def _rendezvous(exp_id: str) -> ExpStore:
    global IS_STORE_HOST, STORE_ADDR, STORE_PORT, _SERVER_PROC
    try:
        meet_dir = os.environ["STEPTRON_MEET_DIR"]
    except KeyError as exc:
        raise RuntimeError("STEPTRON_MEET_DIR is not set; cannot use shared filesystem rendezvous.") from exc
    os.makedirs(meet_dir, exist_ok=True)
    try:
        host = socket.gethostbyname(socket.getfqdn(socket.gethostname()))
    except OSError:
        host = "127.0.0.1"
    me = f"{host}:{os.getpid()}"
    path = os.path.join(meet_dir, f"redis-rendezvous-{exp_id}.pkl")

    def read_state():
        try:
            with open(path, "rb") as f:
                return pickle.load(f)
        except Exception:
            return None

    def write_state(state: dict):
        tmp = f"{path}.{uuid.uuid4().hex}.tmp"
        with open(tmp, "wb") as f:
            pickle.dump(state, f)
        os.replace(tmp, path)

    def stale(state: dict) -> bool:
        created = state.get("created_at")
        if created is None:
            try:
                created = os.path.getmtime(path)
            except OSError:
                return True
        return time.time() - created > 3600 * 24

    def try_claim():
        global _SERVER_PROC
        try:
            os.close(os.open(path, os.O_CREAT | os.O_EXCL | os.O_WRONLY))
        except FileExistsError:
            return None
        state = {"exp_id": exp_id, "master": me, "port": None, "created_at": time.time()}
        write_state(state)
        try:
            _SERVER_PROC, port = start_store_server()
        except Exception:
            try:
                os.remove(path)
            except FileNotFoundError:
                pass
            raise
        state["port"] = port
        write_state(state)
        return port

    cannot_host = os.environ.get("CANNOT_BE_REDIS_SERVER") == "1"
    master = port = None
    t_start, t_port = time.monotonic(), None
    while True:
        state = read_state()
        if state is None and os.path.exists(path):
            # the claimant has created the file but not written it yet (or it is unreadable)
            try:
                if time.time() - os.path.getmtime(path) > 120:
                    os.remove(path)
            except OSError:
                pass
        elif state is not None and stale(state):
            try:
                os.remove(path)
            except FileNotFoundError:
                pass
            state = None
        if state is None:
            if not cannot_host and not os.path.exists(path):
                port = try_claim()
                if port is not None:
                    master, IS_STORE_HOST = me, True
                    break
        else:
            master = state.get("master")
            port = state.get("port")
            if port is not None:
                port = int(port)
                break
            t_port = t_port or time.monotonic()
            if time.monotonic() - t_port > 120:
                raise TimeoutError("Timeout waiting for the store port in the rendezvous file")
        if time.monotonic() - t_start > 3600:
            raise TimeoutError("Timeout waiting for shared filesystem rendezvous")
        time.sleep(0.2)
    STORE_ADDR, STORE_PORT = master.split(":")[0], port
    client = ExpStore(STORE_ADDR, port)
    client.ping()
    return client


def get_exp_redis() -> ExpStore:
    """The experiment store client of this process, creating (or joining) the store on first use."""
    global STORE
    with _LOCK:
        if STORE is None:
            STORE = _rendezvous(f"{{exp}}redis-master-for-{get_exp_id()}")
    return STORE


get_exp_store = get_exp_redis


class AsyncExpStore:
    """``await``-able view of the experiment store for coroutines (generation workers, routers).

    Every store method becomes a coroutine that runs the blocking socket call in the event loop's default executor,
    so a poll of the store never stalls the loop.  The reference offers an ``aioredis`` client for the same purpose
    (utils/comm_utils.py:251-264, used by ``RemoteFuture.aget_result`` at :549-568)."""

    def __init__(self, store: ExpStore):
        self._store = store

    def __getattr__(self, name):
        fn = getattr(self._store, name)
        if not callable(fn):
            return fn

        async def call(*args, **kwargs):
            import asyncio
            import functools

            return await asyncio.get_running_loop().run_in_executor(None, functools.partial(fn, *args, **kwargs))

        call.__name__ = name
        return call


def get_exp_aredis() -> AsyncExpStore:
    """The coroutine view of this thread over the experiment store (one per thread, created on first use)."""
    if getattr(_THREAD_LOCAL, "astore", None) is None or _THREAD_LOCAL.astore._store is not STORE:
        _THREAD_LOCAL.astore = AsyncExpStore(get_exp_redis())
    return _THREAD_LOCAL.astore


def reset_exp_store(stop_server: bool = True) -> None:
    """Forget the client (tests); the hosting process also stops its server."""
    global STORE, IS_STORE_HOST, _SERVER_PROC
    with _LOCK:
        if STORE is not None and IS_STORE_HOST and stop_server:
            STORE.shutdown()
            if _SERVER_PROC is not None:
                try:
                    _SERVER_PROC.wait(timeout=5)
                except Exception:
                    _SERVER_PROC.kill()
        STORE, IS_STORE_HOST, _SERVER_PROC = None, False, None


def _world():
    import torch.distributed as dist

    if dist.is_available() and dist.is_initialized():
        return dist.get_rank(), dist.get_world_size()
    return 0, 1


class RedisQueue:
    """Multi-node FIFO with optional named sub-queues.  Closed once *every* rank has called ``close``."""

    def __init__(self, name: str | None = None):
        from .dist_utils import broadcast_tensors

        self.redis = get_exp_redis()
        self.rank, self.world_size = _world()
        qname = name or str(uuid.uuid4())
        if self.world_size > 1 and name is None:
            qname = broadcast_tensors(qname, src=0, group=None)
        self.qname = qname
        self.counter_key, self.closed_key = qname + "_counter", qname + "_closed"
        self.subqueue_list_key = qname + "_subqueue_list"
        self._closed = self._local_closed = False

    def _build_qname(self, subqueue: str | None = None) -> str:
        return self.qname if subqueue is None else f"{self.qname}:{subqueue}"

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        if self.rank == 0:
            for key in self.redis.keys(self.qname):
                self.redis.expire(key, 3600)

    def register_subqueue(self, subqueue: str) -> None:
        self.redis.zadd(self.subqueue_list_key, {subqueue: 0})

    def put(self, data, subqueue: str | None = None, auto_balance: bool = False) -> bool:
        if auto_balance and subqueue is None:
            sq = self.redis.zpopmin_incr(self.subqueue_list_key)  # least-pushed sub-queue, counted in one step
            subqueue = sq.decode() if sq is not None else None
        elif subqueue is not None:
            self.redis.zincrby(self.subqueue_list_key, 1, subqueue)
        self.redis.lpush(self._build_qname(subqueue), pickle.dumps(data))
        return self.redis.incr(self.counter_key) > 0

    def get(self, subqueue_list: list | None = None):
        for sq in (subqueue_list or [None]):
            raw = self.redis.rpop(self._build_qname(sq))
            if raw is not None:
                self.redis.decr(self.counter_key)
                return pickle.loads(raw)
        raise Empty

    @property
    def closed(self) -> bool:
        if not self._closed:
            self._closed = self.redis.llen(self.closed_key) >= self.world_size
        return self._closed

    def query_closed(self) -> bool:
        return self.closed

    def qsize(self) -> int:
        return int(self.redis.get(self.counter_key) or 0)

    def close(self) -> None:
        assert not self._local_closed, "Cannot close a RedisQueue twice!"
        self.redis.lpush(self.closed_key, self.rank)
        self._local_closed = True


class ReusableDistributor:
    """All ranks pour items in, all ranks draw from the shared pool (order not guaranteed); items can be pushed
    back.  Must be constructed on every rank."""

    def __init__(self, data: Iterable = (), name: str | None = None):
        self.queue = RedisQueue(name)
        self.queue.__enter__()
        self._get_counter = 0
        for d in data:
            self.push_back(d)
        import torch.distributed as dist

        if dist.is_available() and dist.is_initialized():
            dist.barrier()
        self.prefered_subqueue_list = None

    def __iter__(self):
        return self

    def __next__(self):
        try:
            item = self.queue.get(self.prefered_subqueue_list)
        except Empty:
            raise StopIteration from None
        self._get_counter += 1
        return item

    def register_subqueue(self, subqueue: str) -> None:
        self.queue.register_subqueue(subqueue)

    def push_back(self, data, subqueue: str | None = None, auto_balance: bool = False):
        return self.queue.put(data, subqueue, auto_balance)

    @property
    def remains(self) -> int:
        return self.queue.qsize()

    @property
    def closed(self) -> bool:
        return self.queue.closed

    def close(self):
        if not self.queue._local_closed:
            self.queue.close()


class LocalFuture:
    class Pending:
        pass

    def __init__(self):
        self.value = LocalFuture.Pending()

    @property
    def completed(self) -> bool:
        return not isinstance(self.value, LocalFuture.Pending)

    def set_result(self, value) -> None:
        assert not self.completed, "Cannot set result of a completed Future!"
        self.value = value

    def result(self, timeout: float | None = None):
        return self.get_result(timeout)

    def get_result(self, timeout: float | None = None):
        t0 = time.monotonic()
        while not self.completed:
            if timeout is not None and time.monotonic() - t0 >= timeout:
                raise TimeoutError(f"LocalFuture timed out after {timeout} seconds")
            time.sleep(0.02)
        return self.value


class RemoteFuture(LocalFuture):
    """A future any process can complete or await knowing only its ``task_id``; the value travels through
    the experiment store and is removed once read.  Picklable."""

    def __init__(self, task_id: str | None = None, ttl: float = 24 * 3600):
        super().__init__()
        self.task_id = task_id or str(uuid.uuid4())
        self.ttl = ttl

    @property
    def _key(self) -> str:
        return f"remote-future:{self.task_id}"

    def set_result(self, value) -> None:
        store = get_exp_redis()
        store.set(self._key, pickle.dumps(value))
        store.expire(self._key, self.ttl)

    def handle_value(self, raw: bytes):
        """What the bytes in the store stand for: the value, or - for a worker's ``{"status": "error", "error": msg}``
        report - an exception that ``get_result`` raises (reference: utils/comm_utils.py:492-520)."""
        value = pickle.loads(raw)
        if isinstance(value, dict) and value.get("status") == "error":
            return RuntimeError(f"task {self.task_id} failed: {value.get('error', 'unknown worker error')}")
        return value

    def poll(self) -> bool:
        if self.completed:
            return True
        raw = get_exp_redis().get(self._key)
        if raw is None:
            return False
        self.value = self.handle_value(raw)
        get_exp_redis().delete(self._key)
        return True

    def get_result(self, timeout: float | None = None):
        t0 = time.monotonic()
        while not self.poll():
            if timeout is not None and time.monotonic() - t0 >= timeout:
                raise TimeoutError(f"RemoteFuture {self.task_id} timed out after {timeout} seconds")
            time.sleep(0.05)
        if isinstance(self.value, Exception):
            raise self.value
        return self.value

    async def aget_result(self, timeout: float | None = None, interval: float = 0.05):
        """``get_result`` for coroutines: polls through the coroutine view of the store and sleeps on the loop."""
        import asyncio

        store = get_exp_aredis()
        t0 = time.monotonic()
        while not self.completed:
            raw = await store.get(self._key)
            if raw is not None:
                self.value = self.handle_value(raw)
                await store.delete(self._key)
                break
            if timeout is not None and time.monotonic() - t0 >= timeout:
                raise TimeoutError(f"RemoteFuture {self.task_id} timed out after {timeout} seconds")
            await asyncio.sleep(interval)
        if isinstance(self.value, Exception):
            raise self.value
        return self.value

    def __getstate__(self):
        return {"task_id": self.task_id, "ttl": self.ttl}

    def __setstate__(self, state):
        self.task_id, self.ttl = state["task_id"], state.get("ttl", 24 * 3600)
        self.value = LocalFuture.Pending()


def get_ready(futures: list, timeout: float | None = None, min_ready: int = 1) -> tuple[list, list]:
    """Split ``futures`` into (ready, pending), waiting until at least ``min_ready`` are ready."""
    t0 = time.monotonic()
    while True:
        ready = [f for f in futures if (f.poll() if isinstance(f, RemoteFuture) else f.completed)]
        if len(ready) >= min(min_ready, len(futures)) or (timeout is not None and time.monotonic() - t0 >= timeout):
            return ready, [f for f in futures if f not in ready]
        time.sleep(0.05)


def wait_by_finish_order(futures: list) -> Iterable:
    """Yield the futures as they complete."""
    pending = list(futures)
    while pending:
        ready, pending = get_ready(pending)
        yield from ready
