"""Shared serving plumbing: engine submission, incremental detokenisation, delta streams.

All three API dialects (OpenAI chat, Anthropic messages, Responses) render a prompt,
submit it to the engine, and consume the same stream of ``(channel, text)`` deltas where
channel is ``reasoning`` or ``content``; tool-call XML is held back from the content
channel and parsed at the end.

Parity: reference ``src/tilerl/server.py`` -- ``_submit:526``, ``await_or_cancel:313``,
``stream_or_cancel:397``, ``_deltas:794``.
"""
from __future__ import annotations

import asyncio
import os
import time
import uuid
from dataclasses import dataclass, field
from typing import Any, AsyncIterator, Dict, List, Optional, Tuple

from ..engine import Engine, EngineOverloaded, SamplingParams
from . import prompt as P
from .idempotency import RUNNING, KeyRegistry


@dataclass
class ServeContext:
    engine: Engine
    tokenizer: Any
    model_name: str = "tilerl-b200"
    completion_timeout_s: float = float(os.environ.get("TRL_COMPLETION_TIMEOUT_S", "600"))
    health_stuck_s: float = float(os.environ.get("TRL_HEALTH_STUCK_S", "30"))
    pace: bool = False
    pace_depth: int = 0          # items buffered before a paced stream starts releasing
    keepalive_s: float = float(os.environ.get("TRL_SSE_KEEPALIVE_S", "10"))   # silence before a stream pings
    started: float = field(default_factory=time.time)
    keys: KeyRegistry = field(default_factory=KeyRegistry)   # idempotency_key -> run (see idempotency.py)
    orphans: List[Tuple[str, int]] = field(default_factory=list)   # keyed runs whose client left before the end


def overloaded_body(msg: str = "engine overloaded, retry later") -> Dict[str, Any]:
    return {"error": {"message": msg, "type": "overloaded_error", "code": "overloaded"}}


def error_body(msg: str, typ: str = "invalid_request_error", param: Optional[str] = None) -> Dict[str, Any]:
    return {"error": {"message": msg, "type": typ, "param": param, "code": None}}


def new_id(prefix: str) -> str:
    return f"{prefix}-{uuid.uuid4().hex[:24]}"


@dataclass
class Job:
    rid: int
    prompt_tokens: int
    thinking: bool
    stop_texts: Tuple[str, ...]
    tools: Optional[List[Dict[str, Any]]]
    want_logprobs: bool = False
    key: Optional[str] = None       # the request's idempotency_key, if it sent one
    attached: bool = False          # True: this job joined a run that an earlier request with the key started


def _key_of(body: Optional[Dict[str, Any]]) -> Optional[str]:
    key = (body or {}).get("idempotency_key")
    if key is None:
        return None
    if not isinstance(key, str) or not key or len(key) > 256:
        raise P.BadRequest("idempotency_key must be a non-empty string of at most 256 characters", "idempotency_key")
    return key


def submit(ctx: ServeContext, messages: List[Dict[str, Any]], *, tools=None, thinking: bool = True,
           max_tokens: int = 512, body: Optional[Dict[str, Any]] = None, stop=None, seed: Optional[int] = None,
           logprobs: bool = False, think_cap: Optional[int] = None) -> Job:
    text = P.render_chat(messages, tools=tools, enable_thinking=thinking)
    ids = ctx.tokenizer.encode(text)
    s = P.sampling(body or {}, thinking)
    stops = () if stop is None else ((stop,) if isinstance(stop, str) else tuple(stop))
    sp = SamplingParams(max_tokens=int(max_tokens), temperature=s["temperature"], top_p=s["top_p"],
                        top_k=s["top_k"], seed=int(seed) if seed is not None else int(time.time_ns() & 0x7FFFFFFF),
                        stop_texts=stops, logprobs=logprobs, max_think_tokens=think_cap)
    key = _key_of(body)
    sweep_orphans(ctx)
    if key is None:
        return Job(ctx.engine.submit(ids, sp), len(ids), thinking, stops, tools, logprobs)
    with ctx.keys.submit_lock():        # two requests racing with one key start one generation
        e = ctx.keys.lookup(key)
        if e is not None:               # running: wait on the same request; finished: replay the retained result
            return Job(e.rid, e.prompt_tokens, thinking, stops, tools, logprobs, key, True)
        rid = ctx.engine.submit(ids, sp)
        ctx.keys.register(key, rid, len(ids))
    return Job(rid, len(ids), thinking, stops, tools, logprobs, key)


def take(ctx: ServeContext, job: Job):
    """``Engine.take`` for a job: a keyed job's result is kept for the key's other waiters and replays."""
    if job.key is None:
        return ctx.engine.take(job.rid)
    return ctx.keys.take(job.key, job.rid, ctx.engine.take)


def peek(ctx: ServeContext, job: Job) -> Tuple[List[int], bool]:
    """Tokens so far and whether the run is over; a keyed job whose result another waiter already took
    reads the retained copy (the engine no longer knows the request)."""
    if job.key is not None:
        res = ctx.keys.stored(job.key)
        if res is not None:
            return list(res.tokens), True
    toks, done = ctx.engine.peek(job.rid)
    if job.key is not None and done and not toks:
        res = ctx.keys.stored(job.key)
        if res is not None:
            return list(res.tokens), True
    return toks, done


def abandon(ctx: ServeContext, job: Job) -> None:
    """The client went away.  A request without a key is cancelled; a keyed one keeps running, and its
    result is retained so that the client's retry with the same key finds it."""
    if job.key is None:
        ctx.engine.cancel(job.rid)
        ctx.engine.take(job.rid)
    else:
        ctx.orphans.append((job.key, job.rid))
        sweep_orphans(ctx)


def sweep_orphans(ctx: ServeContext) -> None:
    """Move the results of finished keyed runs that nobody waits for out of the engine and into the key
    registry (whose budget bounds them), so that an abandoned run does not stay in the engine's table until
    a retry that may never come.  Called on every submission and whenever a client leaves."""
    if not ctx.orphans:
        return
    left = []
    for key, rid in ctx.orphans:
        toks, done = ctx.engine.peek(rid)
        if done:
            ctx.keys.take(key, rid, ctx.engine.take)
        else:
            left.append((key, rid))
    ctx.orphans[:] = left


def cancel(ctx: ServeContext, job: Job) -> None:
    """Stop the run for good (time-out, stop string reached): a later request with the key runs again."""
    ctx.engine.cancel(job.rid)
    ctx.engine.take(job.rid)
    if job.key is not None:
        ctx.keys.forget(job.key)


def _stable_text(ctx: ServeContext, tokens: List[int]) -> str:
    """Decode, holding back a trailing incomplete UTF-8 sequence."""
    text = ctx.tokenizer.decode(tokens)
    while text.endswith("�"):
        text = text[:-1]
    return text


def _strip_specials(text: str) -> str:
    for s in ("<|im_end|>", "<|endoftext|>"):
        text = text.replace(s, "")
    return text


def _truncate_at_stop(text: str, stops: Tuple[str, ...]) -> Tuple[str, bool]:
    cut = min((text.find(s) for s in stops if s in text), default=-1)
    return (text[:cut], True) if cut >= 0 else (text, False)


def _matched_stop(text: str, stops: Tuple[str, ...]) -> Optional[str]:
    """The stop string that ends the text: the one that occurs first (the longest of those that start there)."""
    hits = [(text.find(s), -len(s), s) for s in stops if s and s in text]
    return min(hits)[2] if hits else None


async def deltas(ctx: ServeContext, job: Job, *, disconnected=None, poll_s: float = 0.01,
                 heartbeat_s: Optional[float] = None) -> AsyncIterator[Tuple[str, str]]:
    """Yield ``(channel, new_text)`` as tokens arrive.  Channels: ``reasoning``, ``content``.
    Text that could still turn into a stop string or a tool-call tag is held back.  With
    ``heartbeat_s`` a ``("ping", "")`` item is yielded whenever that long passed without one, so that a
    long cold prefill does not leave the connection silent (the reference's streams send nothing until
    the completion is whole, ``docs/api-compat-surface.md``)."""
    sent_r = sent_c = 0
    t0 = last = time.monotonic()
    markers = list(job.stop_texts) + ["</think>", "<tool_call>"]
    while True:
        toks, done = peek(ctx, job)
        text = _strip_specials(_stable_text(ctx, toks))
        text, stopped = _truncate_at_stop(text, job.stop_texts)
        closed = "</think>" in text or not job.thinking
        reasoning, answer = P.split_think(text, job.thinking)
        if "<tool_call>" in answer:
            answer = answer[:answer.index("<tool_call>")]
        fin = done or stopped
        if not fin:
            if closed:
                answer = answer[:len(answer) - P.holdback(answer, markers)]
            else:
                reasoning = reasoning[:len(reasoning) - P.holdback(reasoning, markers)]
        if len(reasoning) > sent_r:
            yield "reasoning", reasoning[sent_r:]
            sent_r, last = len(reasoning), time.monotonic()
        if len(answer) > sent_c:
            yield "content", answer[sent_c:]
            sent_c, last = len(answer), time.monotonic()
        if heartbeat_s is not None and not fin and time.monotonic() - last >= heartbeat_s:
            yield "ping", ""
            last = time.monotonic()
        if fin:
            if stopped and not done and job.key is None:
                ctx.engine.cancel(job.rid)     # (a keyed run ends by the engine's own stop-text check)
            return
        if disconnected is not None and await disconnected():
            if job.key is None:
                ctx.engine.cancel(job.rid)     # (the caller's take() that follows finds the result)
            return
        if time.monotonic() - t0 > ctx.completion_timeout_s:
            ctx.engine.cancel(job.rid)
            if job.key is not None:
                ctx.keys.forget(job.key)
            raise TimeoutError("completion timed out")
        await asyncio.sleep(poll_s)


@dataclass
class Final:
    reasoning: str
    content: str
    tool_calls: List[Dict[str, Any]]
    finish_reason: str
    prompt_tokens: int
    completion_tokens: int
    logprobs: List[float]
    tokens: List[int]
    cached_tokens: int = 0
    stop_match: Optional[str] = None      # the stop string that ended the answer, if one did
    reasoning_tokens: int = 0             # tokens of the extracted reasoning span


def finalize(ctx: ServeContext, job: Job, res) -> Final:
    text = _strip_specials(ctx.tokenizer.decode(res.tokens))
    match = _matched_stop(text, job.stop_texts)
    text, stopped = _truncate_at_stop(text, job.stop_texts)
    reasoning, answer = P.split_think(text, job.thinking)
    answer, calls = P.parse_tool_calls(answer, job.tools)
    reason = res.finish_reason
    if reason == "error":
        raise RuntimeError(res.error or "request failed")
    if calls:
        reason = "tool_calls"
    elif stopped:
        reason = "stop"
    return Final(reasoning, answer, calls, reason, res.prompt_tokens, len(res.tokens), list(res.logprobs),
                 list(res.tokens), res.cached_tokens, match if stopped and not calls else None,
                 min(len(res.tokens), len(ctx.tokenizer.encode(reasoning))) if reasoning else 0)


async def complete(ctx: ServeContext, job: Job, disconnected=None) -> Optional[Final]:
    """Wait for the request; ``None`` if the client went away (request cancelled)."""
    t0 = time.monotonic()
    while True:
        res = take(ctx, job)
        if res is not None:
            return finalize(ctx, job, res)
        if disconnected is not None and await disconnected():
            abandon(ctx, job)
            return None
        if time.monotonic() - t0 > ctx.completion_timeout_s:
            cancel(ctx, job)
            raise TimeoutError("completion timed out")
        await asyncio.sleep(0.01)


def health(ctx: ServeContext) -> Tuple[int, Dict[str, Any]]:
    live = ctx.engine.liveness()
    stats = ctx.engine.stats()
    stuck = live["last_progress_age_s"] > ctx.health_stuck_s
    degraded = live["degraded"] is not None
    status = 503 if (stuck or degraded) else 200
    body = {"status": "ok" if status == 200 else ("degraded" if degraded else "stuck"),
            "model": ctx.model_name, "uptime_s": round(time.time() - ctx.started, 1),
            "liveness": live, "stats": stats, "idempotency": ctx.keys.stats()}
    return status, body


def metrics_text(ctx: ServeContext) -> str:
    """``GET /metrics``: the numeric part of ``Engine.stats()`` in the Prometheus text exposition format
    (gauges named ``tilerl_<key>``; nested rows such as the memory table become a ``row`` label).  The
    reference exposes its stats through ``/health`` only; this is the same snapshot for a scraper."""
    live = ctx.engine.liveness()
    lines = []

    def emit(name: str, value, labels: str = "") -> None:
        if isinstance(value, bool):
            value = int(value)
        if isinstance(value, (int, float)):
            lines.append(f"tilerl_{name}{labels} {value}")

    for k, v in sorted(ctx.engine.stats().items()):
        if isinstance(v, dict):
            for row, x in sorted(v.items()):
                label = str(row).replace("\\", "/").replace('"', "'")
                emit(k, x, f'{{row="{label}"}}')
        else:
            emit(k, v)
    emit("last_progress_age_seconds", round(float(live["last_progress_age_s"]), 3))
    emit("degraded", live["degraded"] is not None)
    emit("uptime_seconds", round(time.time() - ctx.started, 1))
    for k, v in sorted(ctx.keys.stats().items()):
        emit(f"idempotency_{k}", v)
    return "\n".join(lines) + "\n"
