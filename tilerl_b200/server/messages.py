"""Anthropic-compatible ``POST /v1/messages``.

Accepts ``system`` (string or text blocks), messages whose content is a string or blocks
(``text`` / ``tool_use`` / ``tool_result`` / ``thinking``), ``max_tokens``, ``thinking``
(``{"type": "enabled", "budget_tokens": n}``), ``tools``, ``tool_choice``,
``stop_sequences``, ``temperature``, ``top_p``, ``stream``.  Streaming follows the event
sequence ``message_start -> content_block_start / content_block_delta /
content_block_stop (per block) -> message_delta -> message_stop`` with ``ping`` allowed.

Parity: reference ``src/tilerl/messages.py`` -- ``MessagesRequest:95``,
``_parse_tool_calls:139``, route ``:309``, SSE ``:346``.
"""
from __future__ import annotations

import asyncio
import json
import time
import os
from typing import Any, Dict, List

from fastapi import Request
from fastapi.responses import JSONResponse, StreamingResponse

from ..engine import EngineOverloaded
from . import core
from . import prompt as P

FIELDS = {"model", "messages", "system", "max_tokens", "thinking", "tools", "tool_choice", "stop_sequences",
          "temperature", "top_p", "top_k", "stream", "metadata", "service_tier", "idempotency_key"}


def to_chat_messages(body: Dict[str, Any]) -> List[Dict[str, Any]]:
    """Anthropic blocks -> the internal chat-message list."""
    out: List[Dict[str, Any]] = []
    system = body.get("system")
    if system:
        out.append({"role": "system", "content": P.content_text(system)})
    for m in body["messages"]:
        role, content = m.get("role"), m.get("content")
        if role not in ("user", "assistant"):
            raise P.BadRequest(f"unknown role {role!r}", "messages")
        if isinstance(content, str):
            out.append({"role": role, "content": content})
            continue
        text, calls, results = [], [], []
        for b in content or []:
            t = b.get("type")
            if t == "text":
                text.append(b.get("text", ""))
            elif t == "tool_use":
                calls.append({"function": {"name": b["name"], "arguments": b.get("input", {})}})
            elif t == "tool_result":
                results.append(P.content_text(b.get("content")))
            elif t in ("thinking", "redacted_thinking"):
                continue  # earlier reasoning is not replayed into the prompt
            else:
                raise P.BadRequest(f"unsupported content block type {t!r}", "messages")
        if role == "assistant":
            out.append({"role": "assistant", "content": "".join(text), "tool_calls": calls})
        else:
            for r in results:
                out.append({"role": "tool", "content": r})
            if text or not results:
                out.append({"role": "user", "content": "".join(text)})
    return out


def _normalise(body: Dict[str, Any]) -> Dict[str, Any]:
    P.refuse_unknown(body, FIELDS)
    if not isinstance(body.get("messages"), list) or not body["messages"]:
        raise P.BadRequest("messages must be a non-empty list", "messages")
    if "max_tokens" not in body:
        raise P.BadRequest("max_tokens is required", "max_tokens")
    th = body.get("thinking") or {"type": "disabled"}
    thinking = th.get("type") == "enabled"
    cap = P.think_cap(None, th.get("budget_tokens")) if thinking else None
    tools = body.get("tools") or None
    tc = body.get("tool_choice") or {}
    if tc.get("type") == "none":
        tools = None
    return dict(thinking=thinking, cap=cap, tools=tools, stream=bool(body.get("stream")),
                max_tokens=int(body["max_tokens"]), stop=body.get("stop_sequences"))


def _stop_reason(f: core.Final) -> str:
    """``tool_use`` first, then ``stop_sequence`` (one of the request's ``stop_sequences`` ended the answer),
    else ``max_tokens`` / ``end_turn``."""
    if f.finish_reason == "tool_calls":
        return "tool_use"
    if f.stop_match is not None:
        return "stop_sequence"
    return {"stop": "end_turn", "length": "max_tokens"}.get(f.finish_reason, "end_turn")


def _usage(prompt_tokens: int, output_tokens: int, cached: int) -> Dict[str, int]:
    """All four fields are always present; tokens served from the prefix cache count as cache reads and are
    left out of ``input_tokens``' uncached remainder as the vendor's accounting does."""
    return {"input_tokens": max(0, prompt_tokens - cached), "output_tokens": output_tokens,
            "cache_creation_input_tokens": 0, "cache_read_input_tokens": cached}


def _blocks(f: core.Final) -> List[Dict[str, Any]]:
    blocks: List[Dict[str, Any]] = []
    if f.reasoning:
        blocks.append({"type": "thinking", "thinking": f.reasoning, "signature": ""})
    if f.content or not f.tool_calls:
        blocks.append({"type": "text", "text": f.content})
    for c in f.tool_calls:
        blocks.append({"type": "tool_use", "id": core.new_id("toolu"), "name": c["name"], "input": c["arguments"]})
    return blocks


def _record(body) -> None:
    """``TRL_MESSAGES_RECORD=<file>``: append every request body as one JSON line (request capture
    for replaying client traffic; reference ``TILERL_MESSAGES_RECORD``, ``src/tilerl/messages.py``)."""
    path = os.environ.get("TRL_MESSAGES_RECORD")
    if not path:
        return
    try:
        with open(path, "a", encoding="utf-8") as f:
            f.write(json.dumps({"t": time.time(), "body": body}) + "\n")
    except OSError:
        pass                      # capture must never fail a request


def mount(app, ctx: core.ServeContext) -> None:
    def err(status: int, typ: str, msg: str):
        return JSONResponse({"type": "error", "error": {"type": typ, "message": msg}}, status_code=status)

    @app.post("/v1/messages/count_tokens")
    async def count_tokens(request: Request):
        """Prompt tokens of a messages body, rendered exactly as ``/v1/messages`` would render it; nothing is
        generated (the vendor's route of that name: agent clients call it to budget their context)."""
        try:
            body = await request.json()
            n = _normalise({**body, "max_tokens": body.get("max_tokens", 1)})
            text = P.render_chat(to_chat_messages(body), tools=n["tools"], enable_thinking=n["thinking"])
            return {"input_tokens": len(ctx.tokenizer.encode(text))}
        except P.BadRequest as e:
            return err(400, "invalid_request_error", str(e))
        except (ValueError, json.JSONDecodeError) as e:
            return err(400, "invalid_request_error", str(e))

    @app.post("/v1/messages")
    async def messages(request: Request):
        try:
            body = await request.json()
            _record(body)
            n = _normalise(body)
            job = core.submit(ctx, to_chat_messages(body), tools=n["tools"], thinking=n["thinking"],
                              max_tokens=n["max_tokens"], body=body, stop=n["stop"], think_cap=n["cap"])
        except P.BadRequest as e:
            return err(400, "invalid_request_error", str(e))
        except EngineOverloaded as e:
            return err(529, "overloaded_error", str(e))
        except (ValueError, json.JSONDecodeError) as e:
            return err(400, "invalid_request_error", str(e))
        mid = core.new_id("msg")
        model = body.get("model") or ctx.model_name

        if not n["stream"]:
            try:
                f = await core.complete(ctx, job, request.is_disconnected)
            except TimeoutError as e:
                return err(504, "timeout_error", str(e))
            except RuntimeError as e:
                return err(500, "api_error", str(e))
            if f is None:
                return err(499, "client_closed", "client closed request")
            return {"id": mid, "type": "message", "role": "assistant", "model": model, "content": _blocks(f),
                    "stop_reason": _stop_reason(f), "stop_sequence": f.stop_match,
                    "usage": _usage(f.prompt_tokens, f.completion_tokens, f.cached_tokens)}

        async def sse():
            def ev(name: str, data: Dict[str, Any]) -> str:
                return f"event: {name}\ndata: {json.dumps(data, ensure_ascii=False)}\n\n"
            yield ev("message_start", {"type": "message_start", "message": {
                "id": mid, "type": "message", "role": "assistant", "model": model, "content": [],
                "stop_reason": None, "stop_sequence": None,
                "usage": _usage(job.prompt_tokens, 0, 0)}})
            index, open_kind = -1, None
            try:
                async for ch, text in core.deltas(ctx, job, disconnected=request.is_disconnected,
                                                  heartbeat_s=ctx.keepalive_s):
                    if ch == "ping":
                        yield ev("ping", {"type": "ping"})
                        continue
                    kind = "thinking" if ch == "reasoning" else "text"
                    if kind != open_kind:
                        if open_kind is not None:
                            yield ev("content_block_stop", {"type": "content_block_stop", "index": index})
                        index += 1
                        open_kind = kind
                        block = {"type": "thinking", "thinking": "", "signature": ""} if kind == "thinking" else {"type": "text", "text": ""}
                        yield ev("content_block_start", {"type": "content_block_start", "index": index,
                                                         "content_block": block})
                    delta = ({"type": "thinking_delta", "thinking": text} if kind == "thinking"
                             else {"type": "text_delta", "text": text})
                    yield ev("content_block_delta", {"type": "content_block_delta", "index": index, "delta": delta})
                if open_kind is not None:
                    yield ev("content_block_stop", {"type": "content_block_stop", "index": index})
                res = None
                for _ in range(500):
                    res = core.take(ctx, job)
                    if res is not None:
                        break
                    await asyncio.sleep(0.01)
                if res is None:
                    return
                f = core.finalize(ctx, job, res)
                for c in f.tool_calls:
                    index += 1
                    yield ev("content_block_start", {"type": "content_block_start", "index": index,
                                                     "content_block": {"type": "tool_use", "id": core.new_id("toolu"),
                                                                       "name": c["name"], "input": {}}})
                    yield ev("content_block_delta", {"type": "content_block_delta", "index": index,
                                                     "delta": {"type": "input_json_delta",
                                                               "partial_json": json.dumps(c["arguments"])}})
                    yield ev("content_block_stop", {"type": "content_block_stop", "index": index})
                yield ev("message_delta", {"type": "message_delta",
                                           "delta": {"stop_reason": _stop_reason(f), "stop_sequence": f.stop_match},
                                           "usage": {"output_tokens": f.completion_tokens}})
                yield ev("message_stop", {"type": "message_stop"})
            except (TimeoutError, RuntimeError) as e:
                yield ev("error", {"type": "error", "error": {"type": "api_error", "message": str(e)}})

        return StreamingResponse(sse(), media_type="text/event-stream")
