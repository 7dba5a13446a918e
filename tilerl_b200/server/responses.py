"""OpenAI Responses API: ``POST /v1/responses``.

``input`` is a string or a list of items (``message`` items with typed content parts,
``function_call`` and ``function_call_output`` items); ``instructions`` becomes the
system turn.  The response carries ``output`` items of type ``reasoning``, ``message``
and ``function_call``; streaming emits sequence-numbered events
(``response.created``, ``response.output_item.added``, ``response.output_text.delta``,
``response.reasoning_summary_text.delta``, ``response.output_item.done``,
``response.completed``).

Parity: reference ``src/tilerl/responses.py`` -- ``ResponsesRequest:60``, route ``:245``,
SSE ``:245-321``.
"""
from __future__ import annotations

import asyncio
import json
import time
from typing import Any, Dict, List

from fastapi import Request
from fastapi.responses import JSONResponse, StreamingResponse

from ..engine import EngineOverloaded
from . import core
from . import prompt as P

FIELDS = {"model", "input", "instructions", "max_output_tokens", "temperature", "top_p", "tools", "tool_choice",
          "reasoning", "stream", "store", "metadata", "parallel_tool_calls", "previous_response_id", "text",
          "truncation", "user", "include", "idempotency_key"}


def to_chat_messages(body: Dict[str, Any]) -> List[Dict[str, Any]]:
    out: List[Dict[str, Any]] = []
    if body.get("instructions"):
        out.append({"role": "system", "content": body["instructions"]})
    inp = body.get("input")
    if isinstance(inp, str):
        out.append({"role": "user", "content": inp})
        return out
    for item in inp or []:
        t = item.get("type", "message")
        if t == "message":
            out.append({"role": item.get("role", "user"), "content": P.content_text(item.get("content"))})
        elif t == "function_call":
            args = item.get("arguments", "{}")
            out.append({"role": "assistant", "content": "",
                        "tool_calls": [{"function": {"name": item["name"], "arguments": args}}]})
        elif t == "function_call_output":
            out.append({"role": "tool", "content": P.content_text(item.get("output"))})
        elif t == "reasoning":
            continue
        else:
            raise P.BadRequest(f"unsupported input item type {t!r}", "input")
    return out


def _tools(body):
    tools = []
    for t in body.get("tools") or []:
        if t.get("type", "function") != "function":
            raise P.BadRequest(f"unsupported tool type {t.get('type')!r}", "tools")
        tools.append({"function": {"name": t["name"], "description": t.get("description", ""),
                                   "parameters": t.get("parameters", {})}})
    return tools or None


def _output_items(f: core.Final) -> List[Dict[str, Any]]:
    items: List[Dict[str, Any]] = []
    if f.reasoning:
        items.append({"type": "reasoning", "id": core.new_id("rs"),
                      "summary": [{"type": "summary_text", "text": f.reasoning}],
                      "content": [{"type": "reasoning_text", "text": f.reasoning}]})   # (older SDKs read `content`)
    if f.content or not f.tool_calls:
        items.append({"type": "message", "id": core.new_id("msg"), "role": "assistant", "status": "completed",
                      "content": [{"type": "output_text", "text": f.content, "annotations": []}]})
    for c in f.tool_calls:
        items.append({"type": "function_call", "id": core.new_id("fc"), "call_id": core.new_id("call"),
                      "name": c["name"], "arguments": json.dumps(c["arguments"]), "status": "completed"})
    return items


def _response(rid: str, model: str, f, status: str, created: int) -> Dict[str, Any]:
    body = {"id": rid, "object": "response", "created_at": created, "model": model, "status": status,
            "output": [] if f is None else _output_items(f), "usage": None, "incomplete_details": None}
    if f is not None:
        body["output_text"] = f.content
        body["usage"] = {"input_tokens": f.prompt_tokens, "output_tokens": f.completion_tokens,
                         "total_tokens": f.prompt_tokens + f.completion_tokens,
                         "input_tokens_details": {"cached_tokens": f.cached_tokens, "cache_write_tokens": 0},
                         "output_tokens_details": {"reasoning_tokens": f.reasoning_tokens}}
        if f.finish_reason == "length":
            body["status"] = "incomplete"
            body["incomplete_details"] = {"reason": "max_output_tokens"}
    return body


def mount(app, ctx: core.ServeContext) -> None:
    @app.post("/v1/responses")
    async def responses(request: Request):
        try:
            body = await request.json()
            P.refuse_unknown(body, FIELDS)
            if body.get("previous_response_id"):
                raise P.BadRequest("previous_response_id is not supported (responses are not stored)",
                                   "previous_response_id")
            effort = (body.get("reasoning") or {}).get("effort")
            thinking = effort != "none" if effort is not None else True
            job = core.submit(ctx, to_chat_messages(body), tools=_tools(body), thinking=thinking,
                              max_tokens=int(body.get("max_output_tokens") or 1024), body=body,
                              think_cap=P.think_cap(effort))
        except P.BadRequest as e:
            return JSONResponse(core.error_body(str(e), param=e.param), status_code=400)
        except EngineOverloaded as e:
            return JSONResponse(core.overloaded_body(str(e)), status_code=503)
        except (ValueError, json.JSONDecodeError) as e:
            return JSONResponse(core.error_body(str(e)), status_code=400)
        rid, created = core.new_id("resp"), int(time.time())
        model = body.get("model") or ctx.model_name

        if not body.get("stream"):
            try:
                f = await core.complete(ctx, job, request.is_disconnected)
            except TimeoutError as e:
                return JSONResponse(core.error_body(str(e), "timeout_error"), status_code=504)
            except RuntimeError as e:
                return JSONResponse(core.error_body(str(e), "server_error"), status_code=500)
            if f is None:
                return JSONResponse(core.error_body("client closed request", "client_closed"), status_code=499)
            return _response(rid, model, f, "completed", created)

        async def sse():
            seq = 0

            def ev(name: str, data: Dict[str, Any]) -> str:
                nonlocal seq
                data = {"type": name, "sequence_number": seq, **data}
                seq += 1
                return f"event: {name}\ndata: {json.dumps(data, ensure_ascii=False)}\n\n"
            yield ev("response.created", {"response": _response(rid, model, None, "in_progress", created)})
            index, open_kind, item_id = -1, None, None
            try:
                async for ch, text in core.deltas(ctx, job, disconnected=request.is_disconnected,
                                                  heartbeat_s=ctx.keepalive_s):
                    if ch == "ping":
                        yield ": keepalive\n\n"          # an SSE comment: clients ignore it, proxies see traffic
                        continue
                    kind = "reasoning" if ch == "reasoning" else "message"
                    if kind != open_kind:
                        if open_kind is not None:
                            yield ev("response.output_item.done", {"output_index": index, "item": {"id": item_id, "type": open_kind}})
                        index += 1
                        open_kind, item_id = kind, core.new_id("rs" if kind == "reasoning" else "msg")
                        yield ev("response.output_item.added", {"output_index": index,
                                                                "item": {"id": item_id, "type": kind}})
                    name = "response.reasoning_summary_text.delta" if kind == "reasoning" else "response.output_text.delta"
                    yield ev(name, {"item_id": item_id, "output_index": index, "content_index": 0, "delta": text})
                if open_kind is not None:
                    yield ev("response.output_item.done", {"output_index": index, "item": {"id": item_id, "type": open_kind}})
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
                    item = {"type": "function_call", "id": core.new_id("fc"), "call_id": core.new_id("call"),
                            "name": c["name"], "arguments": json.dumps(c["arguments"]), "status": "completed"}
                    yield ev("response.output_item.added", {"output_index": index, "item": item})
                    yield ev("response.output_item.done", {"output_index": index, "item": item})
                yield ev("response.completed", {"response": _response(rid, model, f, "completed", created)})
            except (TimeoutError, RuntimeError) as e:
                yield ev("error", {"message": str(e)})

        return StreamingResponse(sse(), media_type="text/event-stream")
