"""Host-side failure detection: per-rank heartbeats in a key-value store and a watchdog.

The reference has no failure detection: a rank that throws exits and its peers block in NCCL
forever (tools/distributed/run_qwen_pp_tp_ppo_trainer.sh:123-128).  Here every rank writes a
heartbeat (a counter that only grows) to a store from a small host thread, so a long step or a
checkpoint write does not look like a dead process; before each step the trainer asks the watchdog
whether a peer went silent or reported a failure, and if so raises ``PeerFailure`` on the host
BEFORE launching further kernels or collectives, so that no GPU work is left waiting.  Silence is
judged on the OBSERVER's monotonic clock (how long since this rank last saw the peer's counter
move), never by comparing wall clocks of two machines.  A peer that has not written its first
beat yet (still building its model) is waited for, not reported.  A failing rank records its
exception in the store on the way out.
The store is a ``torch.distributed.TCPStore`` / ``FileStore`` or the in-memory ``DictStore``
used by tests; nothing here touches a GPU.
"""
from __future__ import annotations

import threading
import time
from typing import Dict, List, Optional


class PeerFailure(RuntimeError):
    def __init__(self, ranks: List[int], reason: str):
        super().__init__(f"ranks {ranks}: {reason}")
        self.ranks, self.reason = ranks, reason


class DictStore:
    """In-process stand-in with the ``set`` / ``get`` / ``check`` subset of a c10d store."""

    def __init__(self):
        self._d: Dict[str, bytes] = {}
        self._lock = threading.Lock()
        self.dropped = set()      # keys a fault-injection test makes unwritable

    def set(self, key: str, value) -> None:
        if key in self.dropped:
            return
        with self._lock:
            self._d[key] = value if isinstance(value, bytes) else str(value).encode()

    def get(self, key: str) -> bytes:
        with self._lock:
            return self._d[key]

    def check(self, keys) -> bool:
        with self._lock:
            return all(k in self._d for k in keys)


class Heartbeat:
    def __init__(self, store, rank: int, world: int, prefix: str = "cverl/hb"):
        self.store, self.rank, self.world, self.prefix = store, rank, world, prefix
        self.count = 0
        self._lock = threading.Lock()
        self._thread: Optional[threading.Thread] = None
        self._halt = threading.Event()
        self._step = -1

    def _key(self, rank: int, what: str) -> str:
        return f"{self.prefix}/{what}/{rank}"

    def beat(self, step: Optional[int] = None) -> None:
        with self._lock:
            self.count += 1
            if step is not None:
                self._step = step
            self.store.set(self._key(self.rank, "beat"), f"{self.count}:{time.time()}:{self._step}")

    def start_background(self, period_s: float) -> None:
        """Beats every ``period_s`` seconds from a daemon thread (host only; touches no GPU) until ``stop``."""
        if self._thread is not None:
            return
        self._halt.clear()

        def loop():
            while not self._halt.wait(period_s):
                try:
                    self.beat()
                except Exception:          # the store went away: the process is shutting down
                    return
        self._thread = threading.Thread(target=loop, name="cverl-heartbeat", daemon=True)
        self._thread.start()

    def stop(self) -> None:
        self._halt.set()
        if self._thread is not None:
            self._thread.join(timeout=5.0)
            self._thread = None

    def report_failure(self, message: str) -> None:
        self.store.set(self._key(self.rank, "fail"), message[:2000])

    def read(self, rank: int):
        key = self._key(rank, "beat")
        if not self.store.check([key]):
            return None
        c, t, s = self.store.get(key).decode().split(":")
        return int(c), float(t), int(s)

    def failure_of(self, rank: int) -> Optional[str]:
        key = self._key(rank, "fail")
        return self.store.get(key).decode() if self.store.check([key]) else None


class Watchdog:
    """Declares a peer lost when its heartbeat is older than ``timeout_s`` or it reported a failure."""

    def __init__(self, heartbeat: Heartbeat, timeout_s: float = 30.0, clock=time.monotonic):
        self.hb, self.timeout_s, self.clock = heartbeat, timeout_s, clock
        self._seen: Dict[int, tuple] = {}      # peer -> (last counter seen, observer time when it last moved)
        self._armed_at = clock()

    def wait_for_peers(self, timeout_s: float, poll_s: float = 0.05) -> None:
        """Blocks until every peer has written its first beat (start-up skew: model construction, weight
        loading); raises ``PeerFailure`` for the ones still missing after ``timeout_s``."""
        deadline = self.clock() + timeout_s
        while True:
            failed = self.failed_ranks()
            if failed:
                raise PeerFailure(sorted(failed), "reported a failure: " + "; ".join(failed.values())[:500])
            missing = [r for r in range(self.hb.world) if r != self.hb.rank and self.hb.read(r) is None]
            if not missing:
                break
            if self.clock() > deadline:
                raise PeerFailure(missing, f"never wrote a first heartbeat within {timeout_s} s")
            time.sleep(poll_s)
        now = self.clock()
        self._armed_at = now
        for r in range(self.hb.world):
            if r != self.hb.rank:
                self._seen[r] = (self.hb.read(r)[0], now)

    def silent_ranks(self) -> List[int]:
        now = self.clock()
        out = []
        for r in range(self.hb.world):
            if r == self.hb.rank:
                continue
            beat = self.hb.read(r)
            if beat is None:
                # no first beat yet: silent only once the grace period since arming has run out
                if now - self._armed_at > self.timeout_s:
                    out.append(r)
                continue
            last = self._seen.get(r)
            if last is None or beat[0] != last[0]:
                self._seen[r] = (beat[0], now)
            elif now - last[1] > self.timeout_s:
                out.append(r)
        return out

    def failed_ranks(self) -> Dict[int, str]:
        return {r: m for r in range(self.hb.world) if r != self.hb.rank and (m := self.hb.failure_of(r)) is not None}

    def check(self) -> None:
        """Call between steps, with no kernel or collective of this rank in flight."""
        failed = self.failed_ranks()
        if failed:
            raise PeerFailure(sorted(failed), "reported a failure: " + "; ".join(failed.values())[:500])
        silent = self.silent_ranks()
        if silent:
            raise PeerFailure(silent, f"no heartbeat for more than {self.timeout_s} s")


def guarded(heartbeat: Heartbeat):
    """Decorator for a rank's main: an escaping exception is published to the peers first."""
    def wrap(fn):
        def inner(*a, **k):
            try:
                return fn(*a, **k)
            except PeerFailure:
                raise
            except BaseException as exc:  # noqa: BLE001 - published, then re-raised
                heartbeat.report_failure(f"{type(exc).__name__}: {exc}")
                raise
        return inner
    return wrap
