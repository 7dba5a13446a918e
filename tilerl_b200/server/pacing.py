"""Stream pacing: smooth bursty token arrival (speculative ticks commit several tokens at
once) into a steady cadence for SSE / WebSocket clients.

``Pacer`` keeps an exponential estimate of the arrival rate and releases queued deltas
no faster than that rate (with a cap on added latency), so text appears evenly.

Parity: reference ``src/tilerl/stream_pacing.py``.
"""
from __future__ import annotations

import time
from collections import deque
from typing import Deque, List, Optional, Tuple


class Pacer:
    def __init__(self, enabled: bool = True, max_delay_s: float = 0.25, alpha: float = 0.2,
                 clock=time.monotonic, depth: int = 0):
        """``depth``: items buffered before the paced release starts (headroom that rides over one stall
        of the producer, e.g. a sparse-KV refresh tick); the wait for it is capped by ``max_delay_s``."""
        self.enabled = enabled
        self.depth = max(0, int(depth))
        self._pushed = 0
        self._first_arrival: Optional[float] = None
        self._started = self.depth == 0
        self.max_delay_s = max_delay_s
        self.alpha = alpha
        self.clock = clock
        self.queue: Deque[Tuple[float, str]] = deque()
        self.rate: Optional[float] = None      # items per second
        self._last_arrival: Optional[float] = None
        self._last_release: Optional[float] = None

    def push(self, items: List[str]) -> None:
        now = self.clock()
        if not items:
            return
        if self._last_arrival is not None:
            dt = max(1e-4, now - self._last_arrival)
            inst = len(items) / dt
            self.rate = inst if self.rate is None else (1 - self.alpha) * self.rate + self.alpha * inst
        self._last_arrival = now
        if self._first_arrival is None:
            self._first_arrival = now
        self._pushed += len(items)
        for it in items:
            self.queue.append((now, it))

    def pop_ready(self, flush: bool = False) -> List[str]:
        """Items that may be sent now.  ``flush`` releases everything (end of stream)."""
        if not self.enabled or flush or self.rate is None:
            out = [it for _, it in self.queue]
            self.queue.clear()
            self._last_release = self.clock()
            return out
        now = self.clock()
        if not self._started:
            first = now if self._first_arrival is None else self._first_arrival
            if self._pushed < self.depth and now - first < self.max_delay_s:
                return []                 # still filling the headroom
            self._started = True
        out: List[str] = []
        gap = 1.0 / max(self.rate, 1e-3)
        while self.queue:
            arrived, it = self.queue[0]
            due = (self._last_release or 0.0) + gap
            if now >= due or now - arrived >= self.max_delay_s:
                out.append(it)
                self.queue.popleft()
                self._last_release = now
            else:
                break
        return out

    def next_wait(self) -> float:
        if not self.queue or not self.enabled or self.rate is None:
            return 0.0
        gap = 1.0 / max(self.rate, 1e-3)
        return max(0.0, min(self.max_delay_s, (self._last_release or 0.0) + gap - self.clock()))
