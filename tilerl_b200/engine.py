"""Continuous-batching engine: ``submit`` / ``poll`` / ``step``.

One model forward per tick.  A tick mixes, in one flat token batch, every
sequence that is decoding (one token each, or a width-W speculative chain) with
as many prefill-chunk tokens as the token budget allows.  Admission is FIFO and
happens only when a GDN state slot and enough KV blocks are free; a prefix hit
adopts refcounted blocks plus the GDN snapshot stored with them.  The engine can
be driven tick by tick from tests and from the GRPO loop, or run as a daemon
thread behind the HTTP server.

Decode-only ticks go through a CUDA-graph runner when one is attached
(:mod:`tilerl_b200.graph`); everything else is an eager forward.

Parity: reference ``src/tilerl/engine.py`` -- ``SamplingParams:517``,
``StepLimits:568``, ``Engine.submit:1097``, ``poll:1195``, ``peek:1229``,
``take:1247``, ``step:1256``, ``_admit:1333``, ``_build_plan:1570``,
``_verify:2625``, ``_commit:2705``, ``cancel:2868``, ``_loop:2895``,
``stats:1711``, liveness ``:1688``.
"""
from __future__ import annotations

import os
import threading
import time
from collections import deque
from dataclasses import dataclass, field
from typing import Callable, Deque, Dict, List, Optional, Sequence, Tuple

import torch

from .batch import Batch
from .kv import GdnStatePool, NoPrefixStore, PagedKvPool, PoolExhausted
from .ops import ref
from .ops.ref import KV_BLOCK


class EngineOverloaded(RuntimeError):
    """Raised by ``submit`` when ``max_inflight`` requests are already queued."""


class RequestFailed(RuntimeError):
    pass


class FatalDeviceError(RuntimeError):
    """The device is gone (OOM / sticky CUDA error): the process should exit so a
    supervisor restarts it."""


FATAL_EXIT_CODE = 11


def fatal_device_exit(msg: str) -> None:  # pragma: no cover - terminates the process
    print(f"FATAL_DEVICE: {msg}", flush=True)
    os._exit(FATAL_EXIT_CODE)


@dataclass
class SamplingParams:
    max_tokens: int = 16
    temperature: float = 0.0
    top_p: float = 1.0
    top_k: int = 0
    seed: int = 0
    stop_ids: Tuple[int, ...] = ()
    stop_texts: Tuple[str, ...] = ()
    logprobs: bool = False
    allowed_ids: Optional[Tuple[int, ...]] = None
    max_think_tokens: Optional[int] = None
    ignore_eos: bool = False

    @property
    def untruncated(self) -> bool:
        """True when samples come from the model's full distribution (on-policy RL)."""
        return self.temperature == 1.0 and self.top_p >= 1.0 and self.top_k == 0 \
            and self.allowed_ids is None


@dataclass
class StepLimits:
    max_batch: int = 64              # sequences per tick
    max_batched_tokens: int = 512    # tokens per tick (prefill chunk budget)
    max_total_tokens: int = 1 << 30  # KV tokens across running sequences
    max_inflight: int = 1024         # waiting + running requests
    prefill_align: int = 64          # prefill chunk widths are multiples of this
    # A long cold fill sharing the engine with other requests takes at most `long_prefill_cap` tokens per
    # tick once its context reaches `long_prefill_min`, so a short request that arrives during the fill
    # waits for a short tick (reference docs/serve-cold-prefill-cap.md: 192 on its shared server, 0 =
    # uncapped for a job that owns the engine).  0 switches the cap off; a fill alone in the engine is
    # never capped.
    long_prefill_cap: int = 0
    long_prefill_min: int = 4096


WAITING, PREFILL, DECODE, DONE = "waiting", "prefill", "decode", "done"


@dataclass
class _Req:
    rid: int
    prompt: List[int]
    params: SamplingParams
    state: str = WAITING
    out: List[int] = field(default_factory=list)
    logprobs: List[float] = field(default_factory=list)
    n_computed: int = 0
    blocks: List[int] = field(default_factory=list)
    slot: int = -1
    finish_reason: Optional[str] = None
    error: Optional[str] = None
    drafts: List[int] = field(default_factory=list)
    think_tokens: int = 0
    in_think: bool = False
    t_submit: float = 0.0
    t_first: float = 0.0
    t_done: float = 0.0
    prefix_tokens: int = 0
    published: bool = False
    n_last_commit: int = 1   # tokens committed by the last tick (valid tap rows for the drafter)
    resumed: int = 0         # > 0: preempted after this many generated tokens; its context is being recomputed

    @property
    def toks(self) -> List[int]:
        return self.prompt + self.out

    @property
    def context(self) -> List[int]:
        """Tokens a prefill has to run before the request can decode: the prompt, or, after a preemption,
        the prompt and every generated token but the last (which is the input of the next decode tick)."""
        return self.prompt if not self.resumed else self.prompt + self.out[:self.resumed - 1]


@dataclass
class Result:
    rid: int
    tokens: List[int]
    logprobs: List[float]
    finish_reason: str
    prompt_tokens: int
    error: Optional[str] = None
    ttft_s: float = 0.0
    total_s: float = 0.0
    cached_tokens: int = 0


class Engine:
    def __init__(self, model, ops, kv_pool: PagedKvPool, state_pool: GdnStatePool, *,
                 limits: Optional[StepLimits] = None, prefix_store=None, eos_id: Optional[int] = None,
                 detokenize: Optional[Callable[[Sequence[int]], str]] = None,
                 think_ids: Optional[Tuple[int, int]] = None, drafter=None, spec_width: int = 0,
                 graph_runner=None, sparse=None, verify_graph_runner=None):
        self.model, self.ops = model, ops
        self.kv, self.states = kv_pool, state_pool
        self.limits = limits or StepLimits()
        self.prefix = prefix_store if prefix_store is not None else NoPrefixStore()
        self.eos_id = eos_id
        self.detok = detokenize
        self.think_ids = think_ids
        self.drafter = drafter
        self.spec_width = spec_width if drafter is not None else 0
        # benchmark seam: count every draft as accepted, to time the verify tick at full acceptance
        # on models whose greedy choice flips with rounding (random-init weights)
        self.spec_force_accept = False
        self._events = 0                      # requests finished or preempted so far (progress without a forward)
        # False: walk the chain on the host even when the verify graph counted the accepted drafts (test seam)
        self.spec_device_accept = True
        self.graph = graph_runner
        self.vgraph = verify_graph_runner       # CUDA-graph replay of width-W verify ticks
        self.sparse = sparse
        self.device = kv_pool.k.device
        self._lock = threading.RLock()
        self._next = 1
        self._waiting: Deque[_Req] = deque()
        self._running: List[_Req] = []
        self._reqs: Dict[int, _Req] = {}
        self._thread: Optional[threading.Thread] = None
        self._stop = threading.Event()
        self._wake = threading.Event()
        self._last_progress = time.monotonic()
        self._degraded: Optional[str] = None
        self.counters = dict(ticks=0, prefill_ticks=0, decode_ticks=0, mixed_ticks=0,
                             graph_ticks=0, tokens_generated=0, prompt_tokens=0,
                             spec_drafted=0, spec_accepted=0, spec_device_accepts=0, cancelled=0, failed=0,
                             finished=0, preempted=0, sparse_ticks=0, dense_ticks=0, verify_ticks=0)
        self.timing = os.environ.get("TRL_STEP_TIMING") == "1"
        # TRL_NVTX=1: every tick and its sampling phase become NVTX ranges, so a profiler can be
        # limited to them (ncu --nvtx --nvtx-include "tick/", nsys --capture-range=nvtx)
        self.nvtx = os.environ.get("TRL_NVTX") == "1" and torch.device(self.device).type == "cuda"
        self.last_tick_ms: Dict[str, float] = {}
        self._memory_rows: Optional[Dict[str, int]] = None
        self.io_h2d = 0   # bytes copied host->device for tick inputs (eager ticks)
        self.io_d2h = 0   # bytes read back (sampled tokens / logits rows)

    # ---- public API -------------------------------------------------------------
    def submit(self, prompt: Sequence[int], params: Optional[SamplingParams] = None) -> int:
        params = params or SamplingParams()
        if len(prompt) == 0:
            raise ValueError("empty prompt")
        if len(prompt) + params.max_tokens > self.model.cfg.max_ctx:
            raise ValueError("prompt + max_tokens exceeds the model context")
        with self._lock:
            if len(self._waiting) + len(self._running) >= self.limits.max_inflight:
                raise EngineOverloaded(f"{self.limits.max_inflight} requests already in flight")
            r = _Req(self._next, [int(t) for t in prompt], params, t_submit=time.monotonic())
            self._next += 1
            self._reqs[r.rid] = r
            self._waiting.append(r)
        self._wake.set()
        return r.rid

    def poll(self, rid: int) -> Dict[str, object]:
        with self._lock:
            r = self._reqs[rid]
            return dict(state=r.state, n_out=len(r.out), finish_reason=r.finish_reason)

    def peek(self, rid: int) -> Tuple[List[int], bool]:
        """Lock-free snapshot of the tokens generated so far (list slicing is atomic
        under the GIL); used by the streaming endpoints."""
        r = self._reqs.get(rid)
        if r is None:
            return [], True
        return r.out[:], r.state == DONE

    def take(self, rid: int) -> Optional[Result]:
        with self._lock:
            r = self._reqs.get(rid)
            if r is None or r.state != DONE:
                return None
            del self._reqs[rid]
            return Result(r.rid, r.out[:], r.logprobs[:], r.finish_reason or "stop", len(r.prompt),
                          r.error, max(0.0, r.t_first - r.t_submit), max(0.0, r.t_done - r.t_submit),
                          r.prefix_tokens)

    def cancel(self, rid: int) -> bool:
        with self._lock:
            r = self._reqs.get(rid)
            if r is None or r.state == DONE:
                return False
            if r in self._waiting:
                self._waiting.remove(r)
            if r in self._running:
                self._running.remove(r)
            self._finish(r, "cancelled")
            self.counters["cancelled"] += 1
            return True

    def has_work(self) -> bool:
        return bool(self._waiting or self._running)

    def generate(self, prompts: Sequence[Sequence[int]], params=None) -> List[Result]:
        """Convenience: submit, drain, return results in order."""
        plist = params if isinstance(params, (list, tuple)) else [params] * len(prompts)
        rids = [self.submit(p, sp) for p, sp in zip(prompts, plist)]
        while any(self._reqs[r].state != DONE for r in rids):
            if not self.step():
                raise RuntimeError("engine stalled with unfinished requests")
        return [self.take(r) for r in rids]

    def invalidate_weights(self) -> None:
        """Weights changed in place: cached KV/prefix content is stale, captured
        graphs stay valid (addresses are unchanged)."""
        with self._lock:
            self.prefix.clear()
            if self.drafter is not None and hasattr(self.drafter, "invalidate"):
                self.drafter.invalidate()
            refresh = getattr(self.ops, "refresh_weight", None)
            if refresh is not None:      # derived device copies of rewritten weights, in place
                for v in self.model.params.values():
                    if hasattr(v, "wq"):
                        refresh(v)

    def precapture(self, batches: Sequence[int] = (1,)) -> None:
        if self.graph is not None:
            self.graph.precapture(batches)

    # ---- liveness / stats ---------------------------------------------------------------
    def liveness(self) -> Dict[str, object]:
        idle = not self.has_work()
        return dict(last_progress_age_s=0.0 if idle else time.monotonic() - self._last_progress,
                    degraded=self._degraded, running=len(self._running), waiting=len(self._waiting))

    def io_bytes(self) -> Tuple[int, int]:
        """(host->device, device->host) bytes moved for tick inputs / sampled tokens."""
        g = self.graph
        return (self.io_h2d + (g.h2d_bytes if g is not None else 0),
                self.io_d2h + (g.d2h_bytes if g is not None else 0))

    def stats(self) -> Dict[str, object]:
        """Lock-free snapshot for ``/health``: queue depths, pool use, prefix and tier traffic, tick counts by
        kind, speculative acceptance, and the bytes the engine's static pools hold (reference
        ``src/tilerl/engine.py:1711``)."""
        out = dict(
            waiting=len(self._waiting), running=len(self._running),
            blocks_used=self.kv.used_blocks, blocks_free=self.kv.free_blocks,
            slots_free=self.states.free_slots,
            prefix_entries=len(self.prefix), prefix_hits=self.prefix.hits,
            prefix_misses=self.prefix.misses, prefix_evictions=self.prefix.evictions,
            **self.counters,
        )
        for k in ("promotions", "demotions", "state_bytes"):
            v = getattr(self.prefix, k, None)
            if v is not None:
                out[f"prefix_{k}"] = int(v)
        drafted = self.counters["spec_drafted"]
        out["spec_acceptance"] = round(self.counters["spec_accepted"] / drafted, 4) if drafted else None
        if self.sparse is not None and isinstance(getattr(self.sparse, "stats", None), dict):
            out["sparse"] = dict(self.sparse.stats)
        if self._memory_rows is None:          # the static pools do not move after construction: measured once
            try:
                from .memory import measure
                self._memory_rows = {k: int(v) for k, v in measure(self).items() if k != "prefix state store"}
            except Exception:  # noqa: BLE001 - a stats call must not fail a health probe
                self._memory_rows = {}
        out["memory"] = dict(self._memory_rows)
        return out

    # ---- daemon loop ----------------------------------------------------------------------
    def run(self, batching_window_s: float = 0.010) -> None:
        if self._thread is not None:
            return
        self._stop.clear()

        def loop():
            last_probe = time.monotonic()
            while not self._stop.is_set():
                if not self.has_work():
                    self._wake.wait(0.05)
                    self._wake.clear()
                    # idle: probe the device now and then, so a dead context is noticed before
                    # the next request pays for it
                    if time.monotonic() - last_probe > 5.0 and hasattr(self.ops, "device_alive"):
                        last_probe = time.monotonic()
                        if not self.ops.device_alive():  # pragma: no cover - needs a dead device
                            self._degraded = "device does not answer"
                            fatal_device_exit(self._degraded)
                    continue
                if not self._running and batching_window_s > 0:
                    time.sleep(batching_window_s)  # let concurrent submits coalesce
                try:
                    self.step()
                except FatalDeviceError as e:  # pragma: no cover
                    self._degraded = str(e)
                    fatal_device_exit(str(e))
                except Exception as e:  # noqa: BLE001 - isolate failures to running rows
                    self._fail_running(repr(e))

        self._thread = threading.Thread(target=loop, name="engine", daemon=True)
        self._thread.start()

    def stop(self) -> None:
        self._stop.set()
        self._wake.set()
        if self._thread is not None:
            self._thread.join(timeout=5)
            self._thread = None

    def _fail_running(self, msg: str) -> None:
        with self._lock:
            for r in list(self._running):
                self._running.remove(r)
                r.error = msg
                self._finish(r, "error")
                self.counters["failed"] += 1

    # ---- one tick ----------------------------------------------------------------------------
    def step(self) -> bool:
        with self._lock:
            t0 = time.perf_counter()
            ev0 = self._events
            self._admit()
            plan = self._build_plan()
            if not plan:
                return self._events != ev0        # nothing to run; a request that was finished or set aside still counts as progress
            t1 = time.perf_counter()
            if self.nvtx:
                torch.cuda.nvtx.range_push(f"tick/{len(plan)}seq/{sum(len(t) for _, t, _ in plan)}tok")
                try:
                    self._run(plan)
                finally:
                    torch.cuda.nvtx.range_pop()
            else:
                self._run(plan)
            self._check_device_error()
            self.counters["ticks"] += 1
            self._last_progress = time.monotonic()
            if self.timing:
                self.last_tick_ms = dict(prep=(t1 - t0) * 1e3, run=(time.perf_counter() - t1) * 1e3)
            return True

    def _check_device_error(self) -> None:
        """A kernel's bounded wait that ran out (a TP peer that never pushed its partial rows, a
        copy that never landed) leaves a record in the device error word and returns: the tick then
        completed on incomplete sums.  Read the word once per tick; on a record, fail the requests
        of this tick instead of emitting their tokens, and tell the caller."""
        read = getattr(self.ops, "read_device_error", None)
        if read is None:
            return
        code, a, b, c = read()
        if code:
            from .parallel.health import CommTimeout
            msg = f"device wait gave up: code={code} a={a} b={b} c={c}"
            self.counters["device_errors"] = self.counters.get("device_errors", 0) + 1
            self._degraded = msg
            self._fail_running(msg)
            raise CommTimeout(msg)

    def _blocks_needed(self, n_tokens: int) -> int:
        return (n_tokens + KV_BLOCK - 1) // KV_BLOCK

    def _admit(self) -> None:
        while self._waiting and len(self._running) < self.limits.max_batch:
            r = self._waiting[0]
            spec_pad = self.spec_width
            need_tokens = len(r.context) + 1 + spec_pad
            hit = self.prefix.lookup(r.context)
            have = len(hit.blocks) if hit else 0
            need = self._blocks_needed(need_tokens) - have
            if self.kv.free_blocks < need:
                self.prefix.evict_until_free(need)
            if self.kv.free_blocks < need or self.states.free_slots < 1:
                if hit:
                    for b in hit.blocks:
                        self.kv.release(b)
                if not self._running:
                    # nothing will ever free memory for it: fail instead of spinning
                    self._waiting.popleft()
                    r.error = "request does not fit in the KV pool"
                    self._finish(r, "error")
                    self.counters["failed"] += 1
                    continue
                break
            self._waiting.popleft()
            r.slot = self.states.alloc_slot()
            if hit:
                r.blocks = list(hit.blocks)
                r.n_computed = r.prefix_tokens = hit.n_tokens
                if hit.snapshot is not None:
                    self.states.restore(r.slot, hit.snapshot)
            for _ in range(need):
                r.blocks.append(self.kv.alloc_block())
            r.state = PREFILL
            self._running.append(r)
            if not r.resumed:
                self.counters["prompt_tokens"] += len(r.prompt)

    def _grow(self, r: _Req, upto_tokens: int) -> bool:
        while len(r.blocks) * KV_BLOCK < upto_tokens:
            if self.kv.free_blocks < 1:
                self.prefix.evict_until_free(1)
            try:
                r.blocks.append(self.kv.alloc_block())
            except PoolExhausted:
                return False
        return True

    def _build_plan(self) -> List[Tuple[_Req, List[int], int]]:
        """[(request, tokens to run this tick, start position)]."""
        plan: List[Tuple[_Req, List[int], int]] = []
        budget = self.limits.max_batched_tokens
        for r in list(self._running):
            if r.state != DECODE:
                continue
            chain = [r.toks[-1]] + (r.drafts if self.spec_width else [])
            start = len(r.toks) - 1
            if not self._grow(r, start + len(chain)):
                # the pool is exhausted: the newest running requests give their pages back and wait to be
                # recomputed; only a request that cannot grow with the pool to itself is cut short
                while not self._grow(r, start + len(chain)):
                    victim = next((v for v in reversed(self._running) if v is not r and v.state in (DECODE, PREFILL)
                                   and all(v is not q for q, _, _ in plan)), None)
                    if victim is None:
                        break
                    self._preempt(victim)
                if not self._grow(r, start + len(chain)):
                    if any(v is not r for v in self._running):
                        self._preempt(r)           # others hold the pool and are already planned: this one waits
                    else:
                        self._running.remove(r)
                        self._finish(r, "length" if r.out else "error")
                        self.counters["failed"] += 0 if r.out else 1
                    continue
            plan.append((r, chain, start))
            budget -= len(chain)
        for r in self._running:
            if r.state != PREFILL or budget <= 0:
                continue
            ctx = r.context
            n_prompt = len(ctx)
            take = budget
            cap = self.limits.long_prefill_cap
            if cap and n_prompt >= self.limits.long_prefill_min and (len(self._running) > 1 or self._waiting):
                take = min(take, max(cap, self.limits.prefill_align))
            end = min(n_prompt, r.n_computed + take)
            if end < n_prompt:
                al = self.limits.prefill_align
                end = max(r.n_computed + 1, r.n_computed + (end - r.n_computed) // al * al)
            boundary = (n_prompt - 1) // KV_BLOCK * KV_BLOCK
            if not isinstance(self.prefix, NoPrefixStore) and r.n_computed < boundary < end \
                    and not r.published and not r.resumed:
                end = boundary  # stop at the block boundary so the GDN snapshot matches it
            toks = ctx[r.n_computed:end]
            plan.append((r, toks, r.n_computed))
            budget -= len(toks)
        return plan

    def _run(self, plan) -> None:
        verify = self.spec_width > 0 and any(r.state == DECODE and len(t) > 1 for r, t, _ in plan)
        decode_only = all(r.state == DECODE for r, _, _ in plan)
        seqs = [dict(tokens=t, start=s, blocks=r.blocks, slot=r.slot,
                     keep=verify and r.state == DECODE) for r, t, s in plan]
        logits = None
        if self.graph is not None and decode_only and not verify and self.sparse is None:
            logits = self.graph.run(seqs)
            if logits is not None:
                self.counters["graph_ticks"] += 1
        taps = hidden = None
        amax = None
        vout = None
        dev_accept = None       # per sequence: drafts accepted, counted (and the state plane selected) on the device
        sparse_tick = False     # True when this tick's attention reads selected pages
        if logits is None and self.vgraph is not None and decode_only and verify and self.sparse is None:
            greedy = all(self._is_plain_greedy(r) for r, _, _ in plan)
            vout = self.vgraph.run(seqs, need_logits=not greedy)
        if vout is not None:
            self.counters["graph_ticks"] += 1
            logits, taps = vout.logits, vout.taps
            amax = vout.argmax if greedy else None
            dev_accept = vout.accept if greedy else None
        elif logits is not None:
            logits, amax = logits.logits, logits.argmax
            if not all(self._is_plain_greedy(r) for r, _, _ in plan):
                amax = None
        else:
            keep = max(len(t) for _, t, _ in plan) if verify else 0
            batch = Batch.build(seqs, self.device, keep_steps=keep)
            self.io_h2d += batch.h2d_bytes
            if self.sparse is not None:
                batch.sparse = self.sparse.for_batch(batch, [r.rid for r, _, _ in plan])
                sparse_tick = batch.sparse is not None
            aux = tuple(self.drafter.aux_layers) if self.drafter is not None else ()
            res = self.model.forward(batch, self.ops, self.kv, self.states,
                                     last_only=not verify, aux_layers=aux)
            if aux:
                logits, hidden, taps = res
            else:
                logits = res
            if all(self._is_plain_greedy(r) for r, _, _ in plan):
                amax = [int(v) for v in self.ops.argmax(logits).tolist()]  # one device sync per tick
                self.io_d2h += 4 * len(amax)
        if amax is None and hasattr(self.ops, "full_logits"):
            logits = self.ops.full_logits(logits)   # sampling needs every vocab shard
        self._presampled = self._presample(plan, logits, verify) if amax is None else {}
        kinds = {r.state for r, _, _ in plan}
        key = "mixed_ticks" if len(kinds) > 1 else ("decode_ticks" if DECODE in kinds else "prefill_ticks")
        self.counters[key] += 1
        self.counters["sparse_ticks" if sparse_tick else "dense_ticks"] += 1
        if verify:
            self.counters["verify_ticks"] += 1
        tok_off = 0
        for i, (r, toks, start) in enumerate(plan):
            n = len(toks)
            base = tok_off if verify else i        # first logits row of this sequence
            last = base + n - 1 if verify else i   # row of its last token
            if r.state == PREFILL:
                r.n_computed = start + n
                if r.resumed:
                    if r.n_computed == len(r.context):       # recomputed: the next tick decodes from its last token
                        r.state, r.resumed = DECODE, 0
                        r.n_computed = len(r.toks) - 1
                else:
                    self._maybe_publish(r)
                    if r.n_computed == len(r.prompt):
                        r.state = DECODE
                        r.t_first = time.monotonic()
                        self._commit(r, [self._sample(r, logits, last, 0, amax)])
                        self._offer_draft(r, taps, tok_off, n)
            else:
                self._verify_commit(r, toks, logits, base, verify, amax,
                                    dev_accept[i] if dev_accept is not None else None)
                self._offer_draft(r, taps, tok_off, n)
            tok_off += n

    # ---- sampling / commit ------------------------------------------------------------------------
    @staticmethod
    def _is_plain_greedy(r: _Req) -> bool:
        p = r.params
        return p.temperature <= 0.0 and p.allowed_ids is None and not p.logprobs \
            and p.max_think_tokens is None

    def _presample(self, plan, logits, verify: bool) -> Dict[int, Tuple[int, float]]:
        """Rows that need seeded temperature sampling, with or without a top-k / top-p restriction,
        are drawn on the device in one kernel when the backend offers it; rows with an allowed-id
        list go through the per-row host sampler."""
        if not hasattr(self.ops, "sample_rows"):
            return {}
        rows, seeds, temps, ks, ps = [], [], [], [], []
        tok_off = 0
        for i, (r, toks, start) in enumerate(plan):
            n = len(toks)
            p = r.params
            base = tok_off if verify else i
            tok_off += n
            if p.temperature <= 0.0 or p.allowed_ids is not None:
                continue
            if r.state == PREFILL:
                if r.resumed or start + n != len(r.prompt):
                    continue
                cand = [(base + n - 1 if verify else i, 0)]
            else:
                cand = [(base + k, k) for k in range(n)] if verify else [(i, 0)]
            for row, k in cand:
                rows.append(row)
                seeds.append(ref.sample_seed(p.seed, len(r.out) + k))
                temps.append(p.temperature)
                ks.append(int(p.top_k or 0))
                ps.append(float(p.top_p))
        if not rows:
            return {}
        toks_, lps = self.ops.sample_rows(logits, rows, seeds, temps, ks, ps)
        self.io_d2h += 8 * len(rows)
        return {row: (int(t), float(lp)) for row, t, lp in zip(rows, toks_, lps)}

    def _sample(self, r: _Req, logits: torch.Tensor, row: int, k: int, amax=None) -> Tuple[int, float]:
        p = r.params
        idx = len(r.out) + k
        if self.think_ids and p.max_think_tokens is not None and r.in_think \
                and r.think_tokens + k >= p.max_think_tokens:
            return self.think_ids[1], 0.0  # forced </think>
        if amax is not None:
            return amax[row], 0.0
        pre = getattr(self, "_presampled", None)
        if pre and row in pre:
            return pre[row]
        allowed = None if p.allowed_ids is None else torch.tensor(p.allowed_ids)
        if p.temperature <= 0.0 and allowed is None and not p.logprobs:
            return int(torch.argmax(logits[row])), 0.0
        return ref.sample(logits[row].detach().float().cpu(), p.temperature, p.top_p, p.top_k,
                          ref.sample_seed(p.seed, idx), allowed)

    def _verify_commit(self, r: _Req, chain: List[int], logits, base: int, verify: bool, amax=None,
                       dev_accept: Optional[int] = None) -> None:
        """``dev_accept``: the verify graph already walked this sequence's chain under greedy acceptance
        and selected the GDN state plane (``spec_accept_kernel``); the host then only commits."""
        on_device = dev_accept is not None and amax is not None and not self.spec_force_accept \
            and self.spec_device_accept and self._is_plain_greedy(r)
        if not verify or len(chain) == 1:
            self._commit(r, [self._sample(r, logits, base, 0, amax)])
            if verify and not on_device:
                self.states.select_step(r.slot, 0)
            return
        drafts = chain[1:]
        if on_device:
            n_ok = int(dev_accept)
            self.counters["spec_drafted"] += len(drafts)
            self.counters["spec_accepted"] += n_ok
            self.counters["spec_device_accepts"] += 1
            self._commit(r, [(amax[base + k], 0.0) for k in range(n_ok + 1)])
            return
        accepted: List[Tuple[int, float]] = []
        n_ok = 0
        for k in range(len(chain)):
            tok = self._sample(r, logits, base + k, k, amax)
            if self.spec_force_accept and k < len(drafts):
                tok = (drafts[k], tok[1])     # timing seam: the draft is taken as the trunk's token
            accepted.append(tok)
            if k < len(drafts) and tok[0] == drafts[k]:
                n_ok += 1
                continue
            break
        self.counters["spec_drafted"] += len(drafts)
        self.counters["spec_accepted"] += n_ok
        # state after the n_ok+1 chain tokens that were really part of the sequence
        self.states.select_step(r.slot, n_ok)
        self._commit(r, accepted)

    def _commit(self, r: _Req, toks: List[Tuple[int, float]]) -> None:
        p = r.params
        r.n_last_commit = len(toks)
        for tok, lp in toks:
            r.out.append(tok)
            if p.logprobs:
                r.logprobs.append(lp)
            self.counters["tokens_generated"] += 1
            if self.think_ids:
                if tok == self.think_ids[0]:
                    r.in_think, r.think_tokens = True, 0
                elif tok == self.think_ids[1]:
                    r.in_think = False
                elif r.in_think:
                    r.think_tokens += 1
            reason = None
            if tok in p.stop_ids or (self.eos_id is not None and tok == self.eos_id and not p.ignore_eos):
                reason = "stop"
            elif p.stop_texts and self.detok is not None:
                text = self.detok(r.out)
                if any(s in text for s in p.stop_texts):
                    reason = "stop"
            if reason is None and len(r.out) >= p.max_tokens:
                reason = "length"
            if reason:
                self._running.remove(r)
                self._finish(r, reason)
                self.counters["finished"] += 1
                return
        r.n_computed = len(r.toks) - 1
        r.drafts = []

    def _offer_draft(self, r: _Req, taps, tok_off: int, n: int) -> None:
        if self.drafter is None or r.state != DECODE:
            return
        r.drafts = self.drafter.propose(self, r, taps, tok_off, n, self.spec_width - 1)

    def _maybe_publish(self, r: _Req) -> None:
        if r.published or isinstance(self.prefix, NoPrefixStore):
            return
        boundary = (len(r.prompt) - 1) // KV_BLOCK * KV_BLOCK
        if boundary and r.n_computed == boundary:
            snap = self.states.snapshot(r.slot) if self.model.cfg.n_gdn_layers else None
            self.prefix.insert(r.prompt[:boundary], r.blocks, snap)
            r.published = True

    def _preempt(self, r: _Req) -> None:
        """Take a running request off the GPU: its KV pages and state slot go back to the pools and it
        returns to the head of the waiting queue; when it is admitted again its context (prompt and the
        tokens generated so far) is recomputed by a prefill and decoding continues where it stopped, so
        the client sees no difference but the delay."""
        self._events += 1
        self._running.remove(r)
        for b in r.blocks:
            self.kv.release(b)
        r.blocks = []
        if r.slot > 0:
            self.states.release(r.slot)
            r.slot = -1
        if self.drafter is not None and hasattr(self.drafter, "release"):
            self.drafter.release(r.rid)
        if self.sparse is not None:
            self.sparse.release(r.rid)
        r.resumed = len(r.out) if r.out else 0
        r.n_computed, r.prefix_tokens, r.drafts, r.state = 0, 0, [], WAITING
        self._waiting.appendleft(r)
        self.counters["preempted"] += 1

    def _finish(self, r: _Req, reason: str) -> None:
        self._events += 1
        r.finish_reason = reason
        r.state = DONE
        r.t_done = time.monotonic()
        for b in r.blocks:
            self.kv.release(b)
        r.blocks = []
        if r.slot > 0:
            self.states.release(r.slot)
            r.slot = -1
        if self.drafter is not None and hasattr(self.drafter, "release"):
            self.drafter.release(r.rid)
        if self.sparse is not None:
            self.sparse.release(r.rid)
