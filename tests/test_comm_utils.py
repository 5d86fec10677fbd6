"""Experiment store: file-system election, the native server's commands, queues and futures."""
import os
import pickle
import threading
from queue import Empty

import pytest


@pytest.fixture()
def store(tmp_path, monkeypatch):
    from steptronoss_b200.utils import comm_utils

    monkeypatch.setenv("STEPTRON_MEET_DIR", str(tmp_path))
    monkeypatch.setenv("EXP_ID", "unit")
    comm_utils.reset_exp_store()
    s = comm_utils.get_exp_redis()
    yield s
    comm_utils.reset_exp_store()


def test_store_commands(store):
    assert store.ping()
    assert store.get("a") is None
    store.set("a", "1")
    assert store.get("a") == b"1" and not store.setnx("a", "2") and store.setnx("b", "2")
    assert store.incr("n") == 1 and store.incr("n", 5) == 6 and store.decr("n") == 5
    for i in range(3):
        store.lpush("q", str(i))
    assert store.llen("q") == 3 and store.rpop("q") == b"0" and store.lpop("q") == b"2"
    assert store.lrange("q") == [b"1"]
    assert sorted(store.keys("")) == [b"a", b"b", b"n", b"q"]
    assert store.delete("a") and store.get("a") is None
    store.zadd("z", {"x": 0, "y": 0})
    first = store.zpopmin_incr("z")
    second = store.zpopmin_incr("z")
    assert {first, second} == {b"x", b"y"}
    big = os.urandom(3 << 20)
    store.set("big", big)
    assert store.get("big") == big
    store.expire("b", 0.0)
    assert store.get("b") is None


def test_election_writes_rendezvous_file_and_second_client_joins(store, tmp_path):
    from steptronoss_b200.utils import comm_utils

    files = [f for f in os.listdir(tmp_path) if f.startswith("redis-rendezvous-")]
    assert len(files) == 1
    state = pickle.load(open(tmp_path / files[0], "rb"))
    assert state["port"] == comm_utils.STORE_PORT and comm_utils.IS_STORE_HOST
    other = comm_utils.ExpStore(comm_utils.STORE_ADDR, state["port"])
    store.set("k", "v")
    assert other.get("k") == b"v"


def test_queue_distributor_and_futures(store):
    from steptronoss_b200.utils.comm_utils import RedisQueue, RemoteFuture, ReusableDistributor, wait_by_finish_order

    q = RedisQueue()
    q.register_subqueue("s0")
    q.register_subqueue("s1")
    for i in range(4):
        q.put(i, auto_balance=True)
    assert q.qsize() == 4
    got = sorted([q.get(["s0"]), q.get(["s0"]), q.get(["s1"]), q.get(["s1"])])
    assert got == [0, 1, 2, 3]
    with pytest.raises(Empty):
        q.get(["s0", "s1", None])
    assert not q.closed
    q.close()
    assert q.closed
    d = ReusableDistributor(range(5))
    seen = [next(d), next(d)]
    d.push_back(seen[0])
    rest = list(d)
    assert sorted(rest + seen[1:]) == [0, 1, 2, 3, 4]
    futs = [RemoteFuture() for _ in range(3)]
    clones = [pickle.loads(pickle.dumps(f)) for f in futs]
    threading.Thread(target=lambda: [c.set_result(i * 10) for i, c in enumerate(clones)]).start()
    assert sorted(f.get_result(timeout=10) for f in wait_by_finish_order(futs)) == [0, 10, 20]
    failed = RemoteFuture()
    pickle.loads(pickle.dumps(failed)).set_result({"status": "error", "error": "out of memory"})     # a worker's report
    with pytest.raises(RuntimeError, match="out of memory"):
        failed.get_result(timeout=10)


def test_coroutines_reach_the_store_without_blocking_the_loop(store):
    import asyncio

    from steptronoss_b200.utils.comm_utils import RemoteFuture, get_exp_aredis

    async def main():
        a = get_exp_aredis()
        assert a is get_exp_aredis()                                    # one view per thread
        await a.set("k", b"v")
        assert await a.get("k") == b"v" and await a.incr("n", 3) == 3
        fut, bad = RemoteFuture(), RemoteFuture()
        ticks = []

        async def ticker():
            while True:
                ticks.append(1)
                await asyncio.sleep(0.01)

        t = asyncio.create_task(ticker())
        threading.Timer(0.15, lambda: pickle.loads(pickle.dumps(fut)).set_result({"x": 1})).start()
        assert await fut.aget_result(timeout=10) == {"x": 1}
        assert len(ticks) >= 3                                          # the loop kept running while the future was polled
        assert store.get(fut._key) is None                              # read once, then removed
        pickle.loads(pickle.dumps(bad)).set_result(ValueError("boom"))
        with pytest.raises(ValueError):
            await bad.aget_result(timeout=10)
        with pytest.raises(TimeoutError):
            await RemoteFuture().aget_result(timeout=0.1)
        t.cancel()

    asyncio.run(main())


def test_blocking_pop_and_score_increments_steer_the_least_loaded_choice(store):
    import time

    assert store.brpop("jobs", timeout=0.1) is None                     # nothing arrives: gives up after the timeout
    threading.Thread(target=lambda: (time.sleep(0.1), store.lpush("jobs", "j1"))).start()
    t0 = time.monotonic()
    assert store.brpop("jobs", timeout=5) == b"j1" and time.monotonic() - t0 < 2
    store.zadd("load", {"a": 0, "b": 0})
    store.zincrby("load", 5, "a")                                       # "a" is busy: the next picks go to "b"
    picks = [store.zpopmin_incr("load") for _ in range(5)]
    assert picks == [b"b"] * 5
    assert {store.zpopmin_incr("load") for _ in range(2)} == {b"a", b"b"}   # both at 5 now: they alternate


def test_safely_start_returns_the_port_of_a_server_that_answers():
    from steptronoss_b200.utils import comm_utils

    comm_utils.reset_exp_store()
    port = comm_utils.safely_start_redis(retries=2, wait_per_retry=0.1)
    try:
        c = comm_utils.ExpStore("127.0.0.1", port, connect_timeout=10)
        assert c.ping() and c.get("redis_start_mark") is None              # the start probe cleaned up after itself
        c.set("k", "v")
        assert c.get("k") == b"v"
    finally:
        c.shutdown()
        if comm_utils._SERVER_PROC is not None:
            comm_utils._SERVER_PROC.wait(timeout=5)
            comm_utils._SERVER_PROC = None
