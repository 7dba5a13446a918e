"""Client-chosen idempotency keys: a retry of the same submission reattaches instead of regenerating.

A request body may carry ``idempotency_key`` (an opaque string, the same field on the chat, messages
and responses routes and on a WebSocket ask; a body field because a WebSocket sends its headers only
once).  The registry sits in front of ``Engine.submit``:

* unknown key: the request runs and the key is bound to its request id (state *running*; only the id
  is held, so in-flight keys cost nothing);
* key of a running request: the caller gets the same request id and waits on it -- no second
  generation, no second block allocation;
* key of a finished request still retained: the stored result is replayed (a request that failed
  replays its error);
* a request that was cancelled, or whose entry was evicted, runs again: the promise is best effort
  inside the retention window, not exactly-once.

``Engine.take`` hands a result to one caller only, so the registry keeps its own copy of a keyed
result: whoever takes it first stores it, every other waiter of the key reads the copy.  Retained
copies are bounded by bytes first (token ids and log-probabilities, 64 MiB by default) and by entry
count second (256); a single result above the per-entry ceiling (16 MiB) is not retained.

The reference describes this behaviour as a design without code
(``docs/design-idempotency-key.md``); the states, budgets and the copy-instead-of-pop rule here follow
that description.
"""
from __future__ import annotations

import threading
import time
from collections import OrderedDict
from dataclasses import dataclass
from typing import Any, Optional

RUNNING, DONE = "running", "done"


@dataclass
class Entry:
    state: str
    rid: int
    prompt_tokens: int
    result: Any = None          # engine.Result once done
    nbytes: int = 0
    born: float = 0.0


def result_bytes(res) -> int:
    """Retained size of a result: 8 bytes per token id and per log-probability (Python's own
    overhead is left out on purpose; the budget bounds the payload, as a token count would)."""
    return 8 * (len(res.tokens) + len(res.logprobs)) + 64


class KeyRegistry:
    def __init__(self, *, max_bytes: int = 64 << 20, max_entries: int = 256, entry_ceiling: int = 16 << 20,
                 max_running: int = 4096):
        self.max_bytes, self.max_entries, self.entry_ceiling = int(max_bytes), int(max_entries), int(entry_ceiling)
        self.max_running = int(max_running)
        self._lock = threading.RLock()
        self._entries: "OrderedDict[str, Entry]" = OrderedDict()
        self._bytes = 0
        self.counters = dict(registered=0, attached=0, replayed=0, evicted=0, oversize=0, dropped=0)

    # ---- submission side --------------------------------------------------------
    def lookup(self, key: str) -> Optional[Entry]:
        with self._lock:
            e = self._entries.get(key)
            if e is not None:
                self.counters["attached" if e.state == RUNNING else "replayed"] += 1
            return e

    def register(self, key: str, rid: int, prompt_tokens: int) -> None:
        with self._lock:
            self._entries[key] = Entry(RUNNING, rid, prompt_tokens, born=time.monotonic())
            self._entries.move_to_end(key)
            self.counters["registered"] += 1
            running = [k for k, e in self._entries.items() if e.state == RUNNING]
            for k in running[:max(0, len(running) - self.max_running)]:      # a bound on abandoned keys
                del self._entries[k]
                self.counters["evicted"] += 1

    def submit_lock(self):
        """Held by the caller across lookup + engine submit + register, so two requests racing with one
        key start one generation."""
        return self._lock

    # ---- completion side --------------------------------------------------------
    def stored(self, key: str):
        with self._lock:
            e = self._entries.get(key)
            return e.result if e is not None and e.state == DONE else None

    def take(self, key: str, rid: int, engine_take):
        """The keyed request's result: the retained copy if there is one, else whatever
        ``engine_take(rid)`` returns, retained for the key's other waiters.  ``None`` while running."""
        with self._lock:
            e = self._entries.get(key)
            if e is not None and e.state == DONE:
                return e.result
            res = engine_take(rid)
            if res is None:
                return None
            if e is None or e.rid != rid:          # evicted meanwhile, or the key now names a newer run
                return res
            if res.finish_reason == "cancelled":   # a retry of a cancelled submission runs again
                del self._entries[key]
                self.counters["dropped"] += 1
                return res
            n = result_bytes(res)
            if n > self.entry_ceiling:
                del self._entries[key]
                self.counters["oversize"] += 1
                return res
            e.state, e.result, e.nbytes, e.born = DONE, res, n, time.monotonic()
            self._entries.move_to_end(key)
            self._bytes += n
            self._evict()
            return res

    def forget(self, key: str) -> None:
        with self._lock:
            e = self._entries.pop(key, None)
            if e is not None:
                self._bytes -= e.nbytes
                self.counters["dropped"] += 1

    def _evict(self) -> None:
        done = [k for k, e in self._entries.items() if e.state == DONE]      # oldest first
        while done and (self._bytes > self.max_bytes or len(done) > self.max_entries):
            e = self._entries.pop(done.pop(0))
            self._bytes -= e.nbytes
            self.counters["evicted"] += 1

    def stats(self) -> dict:
        with self._lock:
            done = sum(1 for e in self._entries.values() if e.state == DONE)
            return dict(self.counters, running=len(self._entries) - done, retained=done, retained_bytes=self._bytes)
