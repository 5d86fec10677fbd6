"""The kernel watchdog (status word and stall detection) and a host model of the peer-memory slot / flag protocol
with threads standing in for ranks."""
import random
import threading
import time

import pytest


def test_watchdog_reports_a_status_code_and_a_stalled_loop():
    from steptronoss_b200.utils.watchdog import KernelWatchdog

    status = {0: 0}
    seen = []
    w = KernelWatchdog(interval_s=0.05, on_error=seen.append, read_status=lambda: dict(status)).start()
    time.sleep(0.2)
    assert not w.tripped.is_set() and seen == []
    status[0] = 5
    assert w.tripped.wait(2.0)
    assert "peer flag wait timed out" in w.error and seen == [w.error]
    with pytest.raises(RuntimeError, match="peer flag"):
        w.raise_if_tripped()
    w.stop()

    seen.clear()
    with KernelWatchdog(interval_s=0.05, stall_s=0.3, on_error=seen.append, read_status=lambda: {0: 0}) as w2:
        for _ in range(5):                       # a loop that beats stays healthy
            time.sleep(0.1)
            w2.beat()
        assert not w2.tripped.is_set()
        assert w2.tripped.wait(3.0)              # ... and one that stops is reported
        assert "no training step finished" in w2.error


class _Rank(threading.Thread):
    """One rank of the exchange used by the peer dispatcher and the fused TP kernels: per call ``e`` it stores a row
    tagged ``e`` into slot ``e % slots`` of every peer, raises its flag to ``e`` on every peer, waits until all of
    its own flags reached ``e`` and then consumes its slot, checking that every row carries exactly ``e``."""

    def __init__(self, me, world, calls, slots, bufs, flags, rng, errors):
        super().__init__(daemon=True)
        self.me, self.world, self.calls, self.slots = me, world, calls, slots
        self.bufs, self.flags, self.rng, self.errors = bufs, flags, rng, errors

    def run(self):
        try:
            for e in range(1, self.calls + 1):
                slot = e % self.slots
                for peer in self.rng.sample(range(self.world), self.world):
                    if self.rng.random() < 0.3:
                        time.sleep(self.rng.random() * 1e-3)
                    self.bufs[peer][slot][self.me] = e           # the data store
                for peer in range(self.world):
                    self.flags[peer][slot][self.me] = e          # the release store, after the data
                deadline = time.time() + 5
                while any(self.flags[self.me][slot][r] < e for r in range(self.world)):
                    if time.time() > deadline:
                        raise TimeoutError(f"rank {self.me} call {e}: flags {self.flags[self.me][slot]}")
                    time.sleep(1e-4)
                if self.rng.random() < 0.3:
                    time.sleep(self.rng.random() * 2e-3)         # a slow consumer
                rows = list(self.bufs[self.me][slot])
                if any(v != e for v in rows):
                    raise AssertionError(f"rank {self.me} call {e} read {rows}")
        except BaseException as ex:  # noqa: BLE001
            self.errors.append(ex)


def _exchange(world, calls, slots, seed):
    bufs = [[[0] * world for _ in range(slots)] for _ in range(world)]
    flags = [[[0] * world for _ in range(slots)] for _ in range(world)]
    errors: list = []
    ranks = [_Rank(r, world, calls, slots, bufs, flags, random.Random(seed * 100 + r), errors) for r in range(world)]
    for t in ranks:
        t.start()
    for t in ranks:
        t.join(60)
    return errors


@pytest.mark.parametrize("world", [2, 4, 8])
def test_two_slots_by_call_parity_are_enough(world):
    """No rank can enter call e before every peer entered call e-1 (it needs their rows of e-1), and a peer that
    entered e-1 has consumed e-2: the slot of parity e is free when call e writes it."""
    for seed in range(2):
        assert _exchange(world, calls=20, slots=2, seed=seed) == []


def test_the_model_detects_a_single_slot_race():
    """With one slot a fast rank overwrites rows of call e with rows of call e+1 before a slow peer has read them."""
    hit = False
    for seed in range(10):
        errs = _exchange(3, calls=40, slots=1, seed=seed)
        if any(isinstance(e, AssertionError) for e in errs):
            hit = True
            break
    assert hit


def test_trainer_stops_when_the_watchdog_sees_a_kernel_error(monkeypatch):
    """A status code that appears while the loop runs ends ``train()`` with that error (host-side injection: the
    status word is a CPU tensor here)."""
    import torch

    from steptronoss_b200.ops import native
    from tests.tiny_exp import make_tiny_exp

    exp = make_tiny_exp(layers=1, hidden=32, heads=2, kv_heads=1, head_dim=16, ffn=64, vocab=64, seq=32, gbs=1, iters=10000)
    exp.profiler_cfg.kernel_watchdog_s = 0.05
    word = torch.zeros(1, dtype=torch.int32)
    monkeypatch.setitem(native._STATUS, 0, word)
    tr = exp.trainer_cfg.get_trainer_cls()(exp=exp)
    threading.Timer(1.0, lambda: word.fill_(4)).start()
    with pytest.raises(RuntimeError, match="epilogue wait timed out"):
        tr.train()
    assert 0 < tr.iteration < 10000
