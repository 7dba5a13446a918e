"""Host-side failure detection for multi-rank jobs.

* :class:`Heartbeat`: every rank publishes a counter in the rendezvous store from a daemon
  thread; :meth:`Heartbeat.check` is called by the training / serving loop *between* steps
  (before the next launch) and raises :class:`PeerLost` when a peer's counter has not moved for
  ``max_age_s`` -- so a rank that died is noticed on the host, not by a collective that never
  returns.  A rank that leaves on purpose calls :meth:`Heartbeat.leave` first.
* :func:`guarded`: run a collective with the process group's (short) timeout turned into a
  :class:`CollectiveTimeout` carrying the step name.
* :func:`order_agrees`: all ranks hash the list of tensor names they are about to reduce and
  compare; a mismatch becomes a message instead of a hang.
* :func:`card_guard`: refuse to start on a GPU that already holds another process's memory.

The GPU side of the story is the device error word: every wait in the fused kernels is bounded
and records ``{code, a, b, c}`` (``ops.native.read_error``); :func:`raise_on_device_error`
turns a recorded word into :class:`CommTimeout` after a step.

Parity: reference ``Backend.device_alive`` (``tilerl_kernels/backend.py:442-465``),
``_order_agrees`` (``src/tilerl/train.py:134-160``), ``card_guard``
(``src/tilerl/engine.py:3000-3052``); the reference has no elastic recovery either (a rank
death aborts the job: ``tests/dp_world4.py:14-16``).
"""
from __future__ import annotations

import hashlib
import threading
import time
from typing import Callable, Dict, List, Optional, Sequence


class PeerLost(RuntimeError):
    def __init__(self, rank: int, age: float):
        super().__init__(f"rank {rank} has not been heard from for {age:.1f} s")
        self.rank, self.age = rank, age


class CollectiveTimeout(RuntimeError):
    pass


class CommTimeout(RuntimeError):
    """A bounded device-side wait ran out (the kernel returned; the context is still usable)."""


class Heartbeat:
    def __init__(self, store, rank: int, world: int, interval_s: float = 0.2, prefix: str = "hb"):
        self.store, self.rank, self.world = store, rank, world
        self.interval, self.prefix = interval_s, prefix
        self._stop = threading.Event()
        self._seen: Dict[int, tuple] = {}
        self._beat = 0
        self._thread = threading.Thread(target=self._run, name="heartbeat", daemon=True)
        self._publish()
        self._thread.start()

    def _key(self, r: int) -> str:
        return f"{self.prefix}/{r}"

    def _publish(self, value: Optional[str] = None) -> None:
        self._beat += 1
        self.store.set(self._key(self.rank), value or str(self._beat))

    def _run(self) -> None:
        while not self._stop.wait(self.interval):
            try:
                self._publish()
            except Exception:  # noqa: BLE001 - the store went away with rank 0: nothing left to tell
                return

    def check(self, max_age_s: float = 2.0) -> None:
        """Raise :class:`PeerLost` for the first peer that stopped beating or left."""
        now = time.monotonic()
        for r in range(self.world):
            if r == self.rank:
                continue
            try:
                val = self.store.get(self._key(r)).decode()
            except Exception:  # noqa: BLE001 - key not there yet: treat as silent since start
                val = ""
            if val == "left":
                raise PeerLost(r, 0.0)
            last = self._seen.get(r)
            if last is None or last[0] != val:
                self._seen[r] = (val, now)
            elif now - last[1] > max_age_s:
                raise PeerLost(r, now - last[1])

    def leave(self) -> None:
        """Announce an orderly exit (between steps, nothing in flight) and stop beating."""
        self._stop.set()
        self._thread.join(timeout=2)
        self.store.set(self._key(self.rank), "left")

    def stop(self) -> None:
        self._stop.set()


def guarded(name: str, fn: Callable, *args, **kw):
    """Call a collective; a process-group timeout becomes :class:`CollectiveTimeout`."""
    try:
        return fn(*args, **kw)
    except RuntimeError as e:
        msg = str(e)
        low = msg.lower()
        if "timeout" in low or "timed out" in low or "connection closed" in low or "reset by peer" in low:
            raise CollectiveTimeout(f"{name}: {msg.splitlines()[0]}") from e
        raise


def order_agrees(names: Sequence[str], group=None) -> bool:
    """True when every rank is about to reduce the same tensors in the same order."""
    import torch
    import torch.distributed as dist
    h = int.from_bytes(hashlib.blake2b("\n".join(names).encode(), digest_size=7).digest(), "big")
    mine = torch.tensor([h], dtype=torch.int64)
    world = dist.get_world_size(group)
    allh = [torch.zeros_like(mine) for _ in range(world)]
    dist.all_gather(allh, mine, group=group)
    return all(int(x) == h for x in allh)


def raise_on_device_error(read_error: Callable[[], Sequence[int]]) -> None:
    code, a, b, c = read_error()
    if code:
        raise CommTimeout(f"device wait gave up: code={code} a={a} b={b} c={c}")


def card_guard(device_index: int = 0, max_foreign_mib: int = 1024, nvml=None) -> None:
    """Refuse a GPU on which other processes already hold more than ``max_foreign_mib``.
    ``nvml``: an object with the pynvml calls used here (tests pass a fake)."""
    import os
    if nvml is None:
        import pynvml as nvml  # type: ignore
        nvml.nvmlInit()
    h = nvml.nvmlDeviceGetHandleByIndex(device_index)
    foreign = 0
    for p in nvml.nvmlDeviceGetComputeRunningProcesses(h):
        if p.pid != os.getpid():
            foreign += int(getattr(p, "usedGpuMemory", 0) or 0)
    if foreign > max_foreign_mib << 20:
        raise RuntimeError(f"GPU {device_index} is in use by other processes ({foreign >> 20} MiB); refusing to start")
