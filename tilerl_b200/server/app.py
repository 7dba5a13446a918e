"""FastAPI application: OpenAI-compatible chat completions plus health, models, a
WebSocket chat channel and a minimal chat page; the Anthropic and Responses dialects are
mounted from their own modules.

Routes: ``GET /health`` (503 when the engine is stuck or degraded), ``GET /v1/models``,
``POST /v1/chat/completions`` (JSON or SSE; ``reasoning_content``, ``tool_calls``,
``logprobs``, ``stream_options.include_usage``), ``WS /ws/chat`` (frames
``delta | tool_calls | done | error``), ``GET /about``, ``GET /chat``.
A client that disconnects cancels its request (logged as 499); an overloaded engine
answers 503 ``overloaded_error``.

Parity: reference ``src/tilerl/server.py`` -- ``ChatCompletionRequest:85``,
``overloaded_body:172``, ``create_app:458``, routes ``:585,:622,:636,:1046,:1150,:1156``,
``_stream:948``; landing page ``src/tilerl/ui_assets.py``.
"""
from __future__ import annotations

import asyncio
import json
import os
import time
from typing import Any, Dict, List, Optional

from fastapi import FastAPI, Request, WebSocket, WebSocketDisconnect
from fastapi.responses import HTMLResponse, JSONResponse, StreamingResponse

from ..engine import EngineOverloaded
from . import core
from . import prompt as P
from .pacing import Pacer

CHAT_FIELDS = {
    "model", "messages", "max_tokens", "max_completion_tokens", "temperature", "top_p", "top_k", "seed", "stop",
    "stream", "stream_options", "logprobs", "top_logprobs", "tools", "tool_choice", "reasoning_effort",
    "chat_template_kwargs", "enable_thinking", "n", "user", "metadata", "presence_penalty",
    "frequency_penalty", "response_format", "parallel_tool_calls", "store", "idempotency_key",
}


def normalise_chat(body: Dict[str, Any]) -> Dict[str, Any]:
    """Validate a chat-completions body; returns the normalised view the handler uses."""
    P.refuse_unknown(body, CHAT_FIELDS)
    if not isinstance(body.get("messages"), list) or not body["messages"]:
        raise P.BadRequest("messages must be a non-empty list", "messages")
    if body.get("n", 1) != 1:
        raise P.BadRequest("only n=1 is supported", "n")
    for k in ("presence_penalty", "frequency_penalty"):
        if body.get(k):
            raise P.BadRequest(f"{k} is not supported", k)
    if body.get("top_logprobs"):
        raise P.BadRequest("top_logprobs is not supported (logprobs returns the sampled token only)", "top_logprobs")
    rf = body.get("response_format")
    if rf and rf.get("type", "text") != "text":
        raise P.BadRequest("only response_format.type == 'text' is supported", "response_format")
    kw = dict(body.get("chat_template_kwargs") or {})
    if "enable_thinking" in body:  # top-level spelling is normalised into the kwargs
        kw["enable_thinking"] = bool(body["enable_thinking"])
    thinking = bool(kw.get("enable_thinking", True))
    effort = body.get("reasoning_effort")
    cap = P.think_cap(effort)
    if effort == "none":
        thinking = False
    max_tokens = body.get("max_completion_tokens") or body.get("max_tokens") or 1024
    if int(max_tokens) < 1:
        raise P.BadRequest("max_tokens must be positive", "max_tokens")
    tools = body.get("tools") or None
    if body.get("tool_choice") == "none":
        tools = None
    return dict(thinking=thinking, cap=cap, max_tokens=int(max_tokens), tools=tools,
                stream=bool(body.get("stream")), include_usage=bool((body.get("stream_options") or {}).get("include_usage")),
                logprobs=bool(body.get("logprobs")), stop=body.get("stop"), seed=body.get("seed"))


def _usage(f: core.Final) -> Dict[str, Any]:
    return {"prompt_tokens": f.prompt_tokens, "completion_tokens": f.completion_tokens,
            "total_tokens": f.prompt_tokens + f.completion_tokens,
            "prompt_tokens_details": {"cached_tokens": f.cached_tokens}}


def _tool_calls_json(calls: List[Dict[str, Any]]) -> List[Dict[str, Any]]:
    return [{"id": core.new_id("call"), "type": "function", "index": i,
             "function": {"name": c["name"], "arguments": json.dumps(c["arguments"], ensure_ascii=False)}}
            for i, c in enumerate(calls)]


def _logprobs_json(ctx, f: core.Final):
    return {"content": [{"token": ctx.tokenizer.decode([t]), "logprob": lp, "bytes": None, "top_logprobs": []}
                        for t, lp in zip(f.tokens, f.logprobs)]}


LANDING = """<!doctype html><html><head><meta charset=utf-8><title>tilerl-b200</title></head>
<body style="font-family:sans-serif;max-width:48rem;margin:2rem auto">
<h1>tilerl-b200</h1><p>Blackwell-native serve-and-train engine. Endpoints:
<code>/v1/chat/completions</code>, <code>/v1/messages</code>, <code>/v1/responses</code>,
<code>/v1/models</code>, <code>/health</code>, <code>/ws/chat</code>. <a href="/chat">Open chat</a>.</p>
</body></html>"""

CHAT_PAGE = """<!doctype html><html><head><meta charset=utf-8><title>chat</title></head>
<body style="font-family:sans-serif;max-width:48rem;margin:1rem auto">
<div id=log style="white-space:pre-wrap;border:1px solid #ccc;padding:.5rem;min-height:20rem"></div>
<form id=f><input id=q style="width:80%" autofocus><button>send</button></form>
<script>
const log=document.getElementById('log'), hist=[];
document.getElementById('f').onsubmit=e=>{e.preventDefault();
 const q=document.getElementById('q'); hist.push({role:'user',content:q.value});
 log.textContent+='\\n> '+q.value+'\\n'; q.value='';
 const ws=new WebSocket((location.protocol=='https:'?'wss://':'ws://')+location.host+'/ws/chat'); let acc='';
 ws.onopen=()=>ws.send(JSON.stringify({messages:hist,max_tokens:512}));
 ws.onmessage=m=>{const f=JSON.parse(m.data);
  if(f.type=='delta'&&f.channel=='content'){acc+=f.text;log.textContent+=f.text;}
  if(f.type=='done'){hist.push({role:'assistant',content:acc});ws.close();}
  if(f.type=='error'){log.textContent+='[error] '+f.message;}};};
</script></body></html>"""


def create_app(engine, tokenizer, model_name: str = "tilerl-b200", *, pace: bool = False, pace_depth: int = 0,
               completion_timeout_s: Optional[float] = None) -> FastAPI:
    ctx = core.ServeContext(engine, tokenizer, model_name, pace=pace, pace_depth=pace_depth)
    if completion_timeout_s is not None:
        ctx.completion_timeout_s = completion_timeout_s
    app = FastAPI(title="tilerl-b200")
    app.state.ctx = ctx

    def bad(e: P.BadRequest):
        return JSONResponse(core.error_body(str(e), param=e.param), status_code=400)

    @app.get("/health")
    async def health():
        status, body = core.health(ctx)
        return JSONResponse(body, status_code=status)

    @app.get("/v1/models")
    async def models():
        return {"object": "list", "data": [{"id": model_name, "object": "model", "created": int(ctx.started),
                                            "owned_by": "tilerl-b200"}]}

    @app.get("/about")
    async def about():
        cfg = engine.model.cfg
        return {"model": model_name, "config": cfg.name, "layers": cfg.n_layers, "hidden": cfg.hidden,
                "quant": cfg.quant, "tp": engine.model.tp}

    @app.get("/", response_class=HTMLResponse)
    async def landing():
        return LANDING

    static_dir = os.path.join(os.path.dirname(os.path.abspath(__file__)), "static")

    @app.get("/chat", response_class=HTMLResponse)
    async def chat_page():
        index = os.path.join(static_dir, "index.html")
        if os.path.exists(index):           # the modular client (ES modules under /static/)
            with open(index, encoding="utf-8") as f:
                return f.read()
        return CHAT_PAGE                     # single-file fallback

    if os.path.isdir(static_dir):
        from fastapi.staticfiles import StaticFiles
        app.mount("/static", StaticFiles(directory=static_dir), name="static")

    @app.get("/metrics")
    async def metrics():
        from fastapi.responses import PlainTextResponse
        return PlainTextResponse(core.metrics_text(ctx), media_type="text/plain; version=0.0.4")

    @app.post("/v1/chat/completions")
    async def chat(request: Request):
        try:
            body = await request.json()
            n = normalise_chat(body)
            job = core.submit(ctx, body["messages"], tools=n["tools"], thinking=n["thinking"],
                              max_tokens=n["max_tokens"], body=body, stop=n["stop"], seed=n["seed"],
                              logprobs=n["logprobs"], think_cap=n["cap"])
        except P.BadRequest as e:
            return bad(e)
        except EngineOverloaded as e:
            return JSONResponse(core.overloaded_body(str(e)), status_code=503)
        except (ValueError, json.JSONDecodeError) as e:
            return JSONResponse(core.error_body(str(e)), status_code=400)
        cid, created = core.new_id("chatcmpl"), int(time.time())

        if not n["stream"]:
            try:
                f = await core.complete(ctx, job, request.is_disconnected)
            except TimeoutError as e:
                return JSONResponse(core.error_body(str(e), "timeout_error"), status_code=504)
            except RuntimeError as e:
                return JSONResponse(core.error_body(str(e), "server_error"), status_code=500)
            if f is None:
                return JSONResponse(core.error_body("client closed request", "client_closed"), status_code=499)
            msg: Dict[str, Any] = {"role": "assistant", "content": f.content or None if f.tool_calls else f.content}
            if f.reasoning:
                msg["reasoning_content"] = f.reasoning
            if f.tool_calls:
                msg["tool_calls"] = _tool_calls_json(f.tool_calls)
            choice = {"index": 0, "message": msg, "finish_reason": f.finish_reason}
            if n["logprobs"]:
                choice["logprobs"] = _logprobs_json(ctx, f)
            return {"id": cid, "object": "chat.completion", "created": created, "model": model_name,
                    "choices": [choice], "usage": _usage(f)}

        async def sse():
            def chunk(delta, finish=None, usage=None, choices=True):
                d = {"id": cid, "object": "chat.completion.chunk", "created": created, "model": model_name,
                     "choices": [{"index": 0, "delta": delta, "finish_reason": finish}] if choices else []}
                if usage is not None:
                    d["usage"] = usage
                return f"data: {json.dumps(d, ensure_ascii=False)}\n\n"
            yield chunk({"role": "assistant", "content": ""})
            pacer = Pacer(enabled=ctx.pace, depth=ctx.pace_depth)
            try:
                async for ch, text in core.deltas(ctx, job, disconnected=request.is_disconnected,
                                                  heartbeat_s=ctx.keepalive_s):
                    if ch == "ping":
                        yield ": keepalive\n\n"          # an SSE comment: clients ignore it, proxies see traffic
                        continue
                    key = "reasoning_content" if ch == "reasoning" else "content"
                    pacer.push([json.dumps({key: text})])
                    for item in pacer.pop_ready():
                        yield chunk(json.loads(item))
                for item in pacer.pop_ready(flush=True):
                    yield chunk(json.loads(item))
                res = None
                for _ in range(500):
                    res = core.take(ctx, job)
                    if res is not None:
                        break
                    await asyncio.sleep(0.01)
                if res is None:
                    return
                f = core.finalize(ctx, job, res)
                if f.tool_calls:
                    yield chunk({"tool_calls": _tool_calls_json(f.tool_calls)})
                yield chunk({}, finish=f.finish_reason)
                if n["include_usage"]:
                    yield chunk({}, usage=_usage(f), choices=False)
                yield "data: [DONE]\n\n"
            except (TimeoutError, RuntimeError) as e:
                yield f"data: {json.dumps(core.error_body(str(e), 'server_error'))}\n\n"

        return StreamingResponse(sse(), media_type="text/event-stream")

    @app.websocket("/ws/chat")
    async def ws_chat(ws: WebSocket):
        await ws.accept()
        try:
            body = json.loads(await ws.receive_text())
            n = normalise_chat({**body, "stream": True})
            job = core.submit(ctx, body["messages"], tools=n["tools"], thinking=n["thinking"],
                              max_tokens=n["max_tokens"], body=body, stop=n["stop"], seed=n["seed"],
                              think_cap=n["cap"])
        except (P.BadRequest, ValueError) as e:
            await ws.send_text(json.dumps({"type": "error", "message": str(e)}))
            await ws.close()
            return
        except EngineOverloaded as e:
            await ws.send_text(json.dumps({"type": "error", "message": str(e), "code": "overloaded"}))
            await ws.close()
            return
        # The socket is read while the answer streams: a {"type": "cancel"} frame stops the run for good
        # (the Stop button), a dropped socket abandons it (a keyed run goes on for the client's retry).
        gone = asyncio.Event()

        async def listen():
            try:
                while True:
                    raw = await ws.receive_text()
                    try:
                        msg = json.loads(raw)
                    except ValueError:
                        continue
                    if isinstance(msg, dict) and msg.get("type") == "cancel":
                        core.cancel(ctx, job)
                        gone.set()
                        return
            except (WebSocketDisconnect, RuntimeError):
                core.abandon(ctx, job)
                gone.set()

        async def disconnected():
            return gone.is_set()

        listener = asyncio.create_task(listen())
        try:
            async for ch, text in core.deltas(ctx, job, disconnected=disconnected):
                await ws.send_text(json.dumps({"type": "delta", "channel": ch, "text": text}))
            res = None
            for _ in range(500):
                if gone.is_set():
                    break
                res = core.take(ctx, job)
                if res is not None:
                    break
                await asyncio.sleep(0.01)
            if res is not None and res.finish_reason != "cancelled":
                f = core.finalize(ctx, job, res)
                if f.tool_calls:
                    await ws.send_text(json.dumps({"type": "tool_calls", "tool_calls": _tool_calls_json(f.tool_calls)}))
                await ws.send_text(json.dumps({"type": "done", "finish_reason": f.finish_reason, "usage": _usage(f)}))
            elif gone.is_set() or res is not None:
                await ws.send_text(json.dumps({"type": "error", "message": "cancelled", "code": "cancelled"}))
        except WebSocketDisconnect:
            core.abandon(ctx, job)
        except (TimeoutError, RuntimeError) as e:
            try:
                await ws.send_text(json.dumps({"type": "error", "message": str(e)}))
            except (WebSocketDisconnect, RuntimeError):
                pass
        finally:
            listener.cancel()

    from .messages import mount as mount_messages
    from .responses import mount as mount_responses
    mount_messages(app, ctx)
    mount_responses(app, ctx)
    return app
