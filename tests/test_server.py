"""API surface over the tiny engine (CPU): raw HTTP through the ASGI app, then the real
``openai`` and ``anthropic`` SDK clients pointed at it."""
import asyncio
import json
import time

import httpx
import pytest

from helpers import make_engine
from tilerl_b200.config import tiny
from tilerl_b200.server.app import create_app
from tilerl_b200.server import prompt as P
from tilerl_b200.tokenizer import ByteTokenizer


@pytest.fixture()
def served():
    eng = make_engine(tiny(max_ctx=2048), blocks=300, slots=6)
    tok = ByteTokenizer()
    eng.eos_id = tok.eos_id
    eng.detok = tok.decode
    eng.think_ids = tok.think_ids
    eng.run(batching_window_s=0.0)
    app = create_app(eng, tok, "tiny-test")
    yield eng, app
    eng.stop()


def _client(app):
    return httpx.AsyncClient(transport=httpx.ASGITransport(app=app), base_url="http://test")


def run(coro):
    return asyncio.run(coro)


def test_prompt_rendering_and_tool_parsing():
    text = P.render_chat([{"role": "system", "content": "be brief"}, {"role": "user", "content": "hi"}],
                         enable_thinking=False)
    assert text.startswith("<|im_start|>system\nbe brief<|im_end|>") and text.endswith("<think>\n\n</think>\n\n")
    assert P.render_chat([{"role": "user", "content": "x"}]).endswith("<|im_start|>assistant\n<think>\n")
    tools = [{"type": "function", "function": {"name": "add", "parameters": {
        "type": "object", "properties": {"a": {"type": "integer"}, "b": {"type": "number"}, "s": {"type": "string"}}}}}]
    assert "<tools>" in P.render_chat([{"role": "user", "content": "x"}], tools=tools)
    out = "ok <tool_call>\n<function=add>\n<parameter=a>\n2\n</parameter>\n<parameter=b>\n1.5\n</parameter>\n" \
          "<parameter=s>\nhey\n</parameter>\n</function>\n</tool_call>"
    rest, calls = P.parse_tool_calls(out, tools)
    assert rest == "ok" and calls == [{"name": "add", "arguments": {"a": 2, "b": 1.5, "s": "hey"}}]
    assert P.split_think("abc</think>\n\nanswer", True) == ("abc", "answer")
    assert P.split_think("still thinking", True) == ("still thinking", "")
    assert P.holdback("hello </thi", ["</think>"]) == 5
    assert P.sampling({}, True)["top_k"] == 20 and P.sampling({"temperature": 0.1}, False)["temperature"] == 0.1
    assert P.think_cap("low") == 512
    with pytest.raises(P.BadRequest):
        P.refuse_unknown({"bogus": 1}, {"model"})


def test_chat_completion_json_health_models(served):
    eng, app = served

    async def go():
        async with _client(app) as c:
            h = await c.get("/health")
            assert h.status_code == 200 and h.json()["status"] == "ok" and "blocks_free" in h.json()["stats"]
            m = await c.get("/v1/models")
            assert m.json()["data"][0]["id"] == "tiny-test"
            r = await c.post("/v1/chat/completions", json={
                "model": "tiny-test", "messages": [{"role": "user", "content": "hello"}], "max_tokens": 12,
                "temperature": 0.0, "top_p": 1.0, "seed": 1, "logprobs": True, "enable_thinking": False})
            assert r.status_code == 200, r.text
            j = r.json()
            ch = j["choices"][0]
            assert j["object"] == "chat.completion" and ch["finish_reason"] in ("stop", "length")
            assert j["usage"]["completion_tokens"] <= 12 and j["usage"]["prompt_tokens"] > 5
            assert len(ch["logprobs"]["content"]) == j["usage"]["completion_tokens"]
            bad = await c.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "x"}], "bogus": 1})
            assert bad.status_code == 400 and "bogus" in bad.json()["error"]["message"]
            bad2 = await c.post("/v1/chat/completions", json={"messages": []})
            assert bad2.status_code == 400
            about = await c.get("/about")
            assert about.json()["layers"] == 2
            assert (await c.get("/chat")).status_code == 200
    run(go())
    assert eng.kv.used_blocks == 0


def test_chat_completion_sse_stream(served):
    eng, app = served

    async def go():
        async with _client(app) as c:
            async with c.stream("POST", "/v1/chat/completions", json={
                    "messages": [{"role": "user", "content": "hi"}], "max_tokens": 10, "stream": True,
                    "stream_options": {"include_usage": True}, "temperature": 0.0}) as r:
                assert r.status_code == 200
                lines = [ln async for ln in r.aiter_lines() if ln.startswith("data: ")]
        assert lines[-1] == "data: [DONE]"
        chunks = [json.loads(ln[6:]) for ln in lines[:-1]]
        assert chunks[0]["choices"][0]["delta"]["role"] == "assistant"
        finishes = [c["choices"][0]["finish_reason"] for c in chunks if c["choices"]]
        assert finishes[-1] in ("stop", "length")
        assert chunks[-1]["usage"]["completion_tokens"] <= 10 and chunks[-1]["choices"] == []
    run(go())


def test_overload_returns_503(served):
    eng, app = served
    eng.limits.max_inflight = 0

    async def go():
        async with _client(app) as c:
            r = await c.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "x"}]})
            assert r.status_code == 503 and r.json()["error"]["type"] == "overloaded_error"
            r2 = await c.post("/v1/messages", json={"model": "m", "max_tokens": 4, "messages": [{"role": "user", "content": "x"}]})
            assert r2.status_code == 529 and r2.json()["error"]["type"] == "overloaded_error"
    run(go())


def test_health_reports_stuck_engine(served):
    eng, app = served
    eng.stop()
    eng.submit([1, 2, 3])
    eng._last_progress -= 1000

    async def go():
        async with _client(app) as c:
            r = await c.get("/health")
            assert r.status_code == 503 and r.json()["status"] == "stuck"
    run(go())


def test_anthropic_messages_json_and_sse(served):
    eng, app = served

    async def go():
        async with _client(app) as c:
            r = await c.post("/v1/messages", json={
                "model": "tiny-test", "max_tokens": 8, "system": "s",
                "messages": [{"role": "user", "content": [{"type": "text", "text": "hi"}]}], "temperature": 0.0})
            assert r.status_code == 200, r.text
            j = r.json()
            assert j["type"] == "message" and j["content"][-1]["type"] == "text"
            assert j["stop_reason"] in ("end_turn", "max_tokens") and j["usage"]["output_tokens"] <= 8
            async with c.stream("POST", "/v1/messages", json={
                    "model": "m", "max_tokens": 8, "stream": True, "thinking": {"type": "enabled", "budget_tokens": 3},
                    "messages": [{"role": "user", "content": "hi"}]}) as s:
                events = [ln[7:] async for ln in s.aiter_lines() if ln.startswith("event: ")]
            assert events[0] == "message_start" and events[-1] == "message_stop" and "message_delta" in events
            assert events.count("content_block_start") == events.count("content_block_stop")
            r3 = await c.post("/v1/messages", json={"model": "m", "messages": [{"role": "user", "content": "x"}]})
            assert r3.status_code == 400 and "max_tokens" in r3.json()["error"]["message"]
    run(go())


def test_responses_api(served):
    eng, app = served

    async def go():
        async with _client(app) as c:
            r = await c.post("/v1/responses", json={"model": "tiny-test", "input": "hello", "max_output_tokens": 8,
                                                    "instructions": "be brief", "reasoning": {"effort": "none"}})
            assert r.status_code == 200, r.text
            j = r.json()
            assert j["object"] == "response" and j["output"][-1]["type"] == "message"
            assert j["usage"]["output_tokens"] <= 8
            # (effort none: no reasoning span, unless the random model happens to emit the closing tag itself)
            assert 0 <= j["usage"]["output_tokens_details"]["reasoning_tokens"] <= j["usage"]["output_tokens"]
            assert j["usage"]["input_tokens_details"] == {"cached_tokens": j["usage"]["input_tokens_details"]["cached_tokens"],
                                                          "cache_write_tokens": 0}
            async with c.stream("POST", "/v1/responses", json={"input": [{"type": "message", "role": "user",
                                "content": [{"type": "input_text", "text": "hi"}]}], "max_output_tokens": 6,
                                "stream": True}) as s:
                datas = [json.loads(ln[6:]) async for ln in s.aiter_lines() if ln.startswith("data: ")]
            assert datas[0]["type"] == "response.created" and datas[-1]["type"] == "response.completed"
            assert [d["sequence_number"] for d in datas] == list(range(len(datas)))
    run(go())
    from tilerl_b200.server import core, responses
    ctx = app.state.ctx
    res = _res(0)
    res.tokens = ctx.tokenizer.encode("<think>\nsome thought</think>\n\nthe answer")
    f = core.finalize(ctx, core.Job(1, 5, True, (), None), res)
    body = responses._response("resp-1", "m", f, "completed", 0)
    item = body["output"][0]
    assert item["type"] == "reasoning" and item["summary"][0] == {"type": "summary_text", "text": f.reasoning}
    assert item["content"][0] == {"type": "reasoning_text", "text": f.reasoning}
    n = body["usage"]["output_tokens_details"]["reasoning_tokens"]
    assert n == len(ctx.tokenizer.encode(f.reasoning)) and 0 < n < body["usage"]["output_tokens"]


def test_real_sdk_clients(served):
    eng, app = served
    import anthropic
    import openai

    async def go():
        http = _client(app)
        oa = openai.AsyncOpenAI(api_key="x", base_url="http://test/v1", http_client=http)
        r = await oa.chat.completions.create(model="tiny-test", messages=[{"role": "user", "content": "hi"}],
                                             max_tokens=6, temperature=0.0)
        assert r.choices[0].finish_reason in ("stop", "length") and r.usage.completion_tokens <= 6
        stream = await oa.chat.completions.create(model="tiny-test", messages=[{"role": "user", "content": "hi"}],
                                                  max_tokens=6, stream=True)
        n = 0
        async for ch in stream:
            n += 1
        assert n >= 2
        models = await oa.models.list()
        assert models.data[0].id == "tiny-test"
        an = anthropic.AsyncAnthropic(api_key="x", base_url="http://test", http_client=_client(app))
        m = await an.messages.create(model="tiny-test", max_tokens=6, messages=[{"role": "user", "content": "hi"}])
        assert m.role == "assistant" and m.usage.output_tokens <= 6
        async with an.messages.stream(model="tiny-test", max_tokens=6,
                                      messages=[{"role": "user", "content": "hi"}]) as st:
            final = await st.get_final_message()
        assert final.stop_reason in ("end_turn", "max_tokens")
    run(go())


def test_websocket_chat(served):
    eng, app = served
    from starlette.testclient import TestClient
    with TestClient(app) as tc:
        with tc.websocket_connect("/ws/chat") as ws:
            ws.send_text(json.dumps({"messages": [{"role": "user", "content": "hi"}], "max_tokens": 5}))
            frames = []
            while True:
                f = json.loads(ws.receive_text())
                frames.append(f)
                if f["type"] in ("done", "error"):
                    break
        assert frames[-1]["type"] == "done" and frames[-1]["usage"]["completion_tokens"] <= 5


def test_stream_pacing():
    from tilerl_b200.server.pacing import Pacer
    t = [0.0]
    p = Pacer(enabled=True, max_delay_s=0.5, clock=lambda: t[0])
    p.push(["a"])
    assert p.pop_ready() == ["a"]
    t[0] = 0.1
    p.push(["b", "c", "d", "e"])          # a burst of 4 in 0.1 s -> 40/s
    first = p.pop_ready()
    assert 1 <= len(first) < 4            # not all at once
    t[0] = 1.0
    assert "".join(first + p.pop_ready()) == "bcde"
    assert Pacer(enabled=False).pop_ready() == []
    # headroom: nothing leaves until `depth` items arrived (or the wait cap ran out), then the usual cadence
    t[0] = 0.0
    p = Pacer(enabled=True, max_delay_s=0.5, clock=lambda: t[0], depth=3)
    p.push(["a"])
    t[0] = 0.05
    p.push(["b"])
    assert p.pop_ready() == []
    t[0] = 0.10
    p.push(["c"])
    got = p.pop_ready()
    assert got and got[0] == "a"
    t[0] = 2.0
    assert "".join(got + p.pop_ready()) == "abc"
    t[0] = 0.0
    p = Pacer(enabled=True, max_delay_s=0.5, clock=lambda: t[0], depth=10)
    p.push(["x"])
    t[0] = 0.1
    p.push(["y"])
    assert p.pop_ready() == []
    t[0] = 0.7                                  # the cap: a short stream is not held back for ever
    assert p.pop_ready()[0] == "x"
    assert Pacer(enabled=True, depth=5).pop_ready(flush=True) == []


def test_web_client_modules_are_served(served):
    eng, app = served

    async def go():
        async with _client(app) as client:
            page = await client.get("/chat")
            assert page.status_code == 200 and "/static/main.js" in page.text
            for mod in ("protocol.js", "transport.js", "streamBuffer.js", "render.js", "meter.js", "main.js"):
                r = await client.get("/static/" + mod)
                assert r.status_code == 200 and ("export" in r.text or "import" in r.text), mod
            proto = (await client.get("/static/protocol.js")).text
            for frame in ("delta", "tool_calls", "done", "error"):
                assert f'"{frame}"' in proto

    run(go())


def test_messages_request_capture(served, tmp_path, monkeypatch):
    eng, app = served
    rec = tmp_path / "req.jsonl"
    monkeypatch.setenv("TRL_MESSAGES_RECORD", str(rec))

    async def go():
        async with _client(app) as client:
            r = await client.post("/v1/messages", json={"model": "m", "max_tokens": 4,
                                                        "messages": [{"role": "user", "content": "hi"}]})
            assert r.status_code == 200

    run(go())
    lines = rec.read_text().splitlines()
    assert len(lines) == 1 and json.loads(lines[0])["body"]["max_tokens"] == 4


# ---- idempotency keys --------------------------------------------------------------------------
def _res(n, reason="stop"):
    from tilerl_b200.engine import Result
    return Result(1, list(range(n)), [0.0] * n, reason, 3)


def test_key_registry_budgets_and_states():
    from tilerl_b200.server.idempotency import KeyRegistry, result_bytes
    reg = KeyRegistry(max_bytes=3 * result_bytes(_res(100)), max_entries=8, entry_ceiling=result_bytes(_res(500)))
    box = {}
    reg.register("a", 1, 3)
    assert reg.lookup("a").state == "running" and reg.take("a", 1, box.get) is None     # nothing finished yet
    box[1] = _res(100)
    first = reg.take("a", 1, lambda rid: box.pop(rid, None))
    again = reg.take("a", 1, lambda rid: box.pop(rid, None))           # the engine gave it away; the copy replays
    assert first is again and reg.lookup("a").state == "done" and reg.stored("a") is first
    for i, k in enumerate("bcd"):                                      # byte budget: the oldest finished entry goes
        reg.register(k, 10 + i, 3)
        reg.take(k, 10 + i, lambda rid: _res(100))
    assert reg.lookup("a") is None and reg.lookup("d") is not None and reg.stats()["retained"] == 3
    reg.register("big", 20, 3)                                          # above the per-entry ceiling: not retained
    assert len(reg.take("big", 20, lambda rid: _res(501)).tokens) == 501 and reg.lookup("big") is None
    reg.register("gone", 21, 3)                                         # a cancelled run is not replayed
    assert reg.take("gone", 21, lambda rid: _res(2, "cancelled")).finish_reason == "cancelled"
    assert reg.lookup("gone") is None
    small = KeyRegistry(max_entries=2)                                  # entry count is the second bound
    for i in range(4):
        small.register(str(i), i, 1)
        small.take(str(i), i, lambda rid: _res(1))
    assert small.stats()["retained"] == 2 and small.lookup("3") is not None and small.lookup("0") is None
    s = reg.stats()
    assert s["oversize"] == 1 and s["dropped"] == 1 and s["evicted"] >= 1 and s["retained_bytes"] <= reg.max_bytes


def test_idempotency_key_replays_and_joins_instead_of_generating_again(served):
    eng, app = served
    ask = {"messages": [{"role": "user", "content": "tell me"}], "max_tokens": 10, "temperature": 1.0,
           "enable_thinking": False}

    async def go():
        async with _client(app) as c:
            a = (await c.post("/v1/chat/completions", json={**ask, "idempotency_key": "k1"})).json()
            done = eng.counters["finished"]
            b = (await c.post("/v1/chat/completions", json={**ask, "idempotency_key": "k1"})).json()
            assert eng.counters["finished"] == done                     # nothing ran for the retry
            assert a["choices"][0]["message"] == b["choices"][0]["message"] and a["usage"] == b["usage"]
            # the retry may come back as a stream: the retained answer arrives as one completed stream
            text = ""
            async with c.stream("POST", "/v1/chat/completions", json={**ask, "idempotency_key": "k1", "stream": True}) as r:
                async for line in r.aiter_lines():
                    if line.startswith("data: {"):
                        for ch in json.loads(line[6:])["choices"]:
                            text += ch["delta"].get("content") or ""
            # (random bytes: the stream holds back an unfinished UTF-8 tail or tag that the whole answer shows)
            norm = lambda t: "".join(ch for ch in t if ch != "\ufffd" and not ch.isspace())
            assert norm(a["choices"][0]["message"]["content"] or "").startswith(norm(text))
            assert eng.counters["finished"] == done
            # two requests racing with one key: one generation, two equal answers
            x, y = await asyncio.gather(c.post("/v1/chat/completions", json={**ask, "idempotency_key": "k2"}),
                                        c.post("/v1/chat/completions", json={**ask, "idempotency_key": "k2"}))
            assert x.status_code == y.status_code == 200 and eng.counters["finished"] == done + 1
            assert x.json()["choices"][0]["message"] == y.json()["choices"][0]["message"]
            # the other dialects take the same field; a key of the wrong type is refused
            m = {"model": "m", "max_tokens": 8, "messages": [{"role": "user", "content": "hi"}], "idempotency_key": "k3"}
            m1, m2 = (await c.post("/v1/messages", json=m)).json(), (await c.post("/v1/messages", json=m)).json()
            assert m1["content"] == m2["content"] and eng.counters["finished"] == done + 2
            r1 = await c.post("/v1/responses", json={"input": "hi", "max_output_tokens": 8, "idempotency_key": "k4"})
            r2 = await c.post("/v1/responses", json={"input": "hi", "max_output_tokens": 8, "idempotency_key": "k4"})
            assert r1.status_code == r2.status_code == 200 and eng.counters["finished"] == done + 3
            bad = await c.post("/v1/chat/completions", json={**ask, "idempotency_key": 7})
            assert bad.status_code == 400 and "idempotency_key" in bad.json()["error"]["message"]
            h = (await c.get("/health")).json()["idempotency"]
            assert h["retained"] == 4 and h["replayed"] >= 4 and h["attached"] + h["replayed"] >= 5
    run(go())
    assert eng.kv.used_blocks == 0


def test_messages_stop_sequence_usage_fields_and_keepalive(served):
    eng, app = served
    from tilerl_b200.server import core, messages
    ctx = app.state.ctx
    tok = ctx.tokenizer
    # the matched stop string: the first to occur; reported as stop_reason "stop_sequence"
    job = core.Job(1, 7, False, ("END", "ZZ"), None)
    res = _res(0)
    res.tokens = tok.encode("alpha ZZ beta END")
    f = core.finalize(ctx, job, res)
    assert f.content == "alpha" and f.stop_match == "ZZ" and messages._stop_reason(f) == "stop_sequence"
    res.tokens = tok.encode("no stop here")
    f = core.finalize(ctx, job, res)
    assert f.stop_match is None and messages._stop_reason(f) == "end_turn"
    assert messages._usage(10, 4, 6) == {"input_tokens": 4, "output_tokens": 4, "cache_creation_input_tokens": 0,
                                         "cache_read_input_tokens": 6}
    ctx.keepalive_s = 0.0            # every poll without new text pings

    async def go():
        async with _client(app) as c:
            j = (await c.post("/v1/messages", json={"model": "m", "max_tokens": 6,
                                                    "messages": [{"role": "user", "content": "hi"}]})).json()
            assert set(j["usage"]) == {"input_tokens", "output_tokens", "cache_creation_input_tokens",
                                       "cache_read_input_tokens"} and j["stop_sequence"] is None
            async with c.stream("POST", "/v1/messages", json={"model": "m", "max_tokens": 40, "stream": True,
                                                              "messages": [{"role": "user", "content": "hi"}]}) as s:
                lines = [ln async for ln in s.aiter_lines()]
            events = [ln[7:] for ln in lines if ln.startswith("event: ")]
            assert "ping" in events and events[0] == "message_start" and events[-1] == "message_stop"
            start = json.loads(next(ln for ln in lines if ln.startswith("data: ") and "message_start" in ln)[6:])
            assert start["message"]["usage"]["output_tokens"] == 0 and "cache_read_input_tokens" in start["message"]["usage"]
            async with c.stream("POST", "/v1/chat/completions", json={
                    "messages": [{"role": "user", "content": "hi"}], "max_tokens": 40, "stream": True}) as s:
                raw = [ln async for ln in s.aiter_lines()]
            assert any(ln.startswith(": keepalive") for ln in raw) and raw[-2 if raw[-1] == "" else -1] == "data: [DONE]"
    run(go())


def test_an_abandoned_keyed_run_finishes_and_its_result_waits_in_the_registry(served):
    eng, app = served
    from tilerl_b200.server import core
    ctx = app.state.ctx
    job = core.submit(ctx, [{"role": "user", "content": "hi"}], max_tokens=6, thinking=False,
                      body={"idempotency_key": "left"})
    core.abandon(ctx, job)                               # the client went away mid-run: the run goes on
    assert ctx.keys.lookup("left") is not None
    for _ in range(500):
        if eng.peek(job.rid)[1]:
            break
        time.sleep(0.01)
    again = core.submit(ctx, [{"role": "user", "content": "hi"}], max_tokens=6, thinking=False,
                        body={"idempotency_key": "left"})      # the retry: sweeps, then replays
    assert again.attached and again.rid == job.rid and not ctx.orphans
    assert job.rid not in eng._reqs                      # the engine no longer holds the finished request
    res = core.take(ctx, again)
    assert res is not None and res.finish_reason in ("stop", "length") and eng.kv.used_blocks == 0


def test_metrics_route_exposes_the_stats_snapshot_as_prometheus_text(served):
    eng, app = served

    async def go():
        async with _client(app) as c:
            await c.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "hi"}], "max_tokens": 4})
            r = await c.get("/metrics")
            assert r.status_code == 200 and r.headers["content-type"].startswith("text/plain")
            return r.text
    text = run(go())
    rows = dict(ln.rsplit(" ", 1) for ln in text.strip().splitlines())
    assert float(rows["tilerl_finished"]) >= 1 and float(rows["tilerl_tokens_generated"]) >= 1
    assert float(rows['tilerl_memory{row="kv pool"}']) > 0 and rows["tilerl_degraded"] == "0"
    assert "tilerl_idempotency_retained" in rows and "tilerl_blocks_free" in rows
    assert all(ln.startswith("tilerl_") for ln in text.strip().splitlines())


def test_messages_count_tokens_matches_what_a_request_is_charged(served):
    eng, app = served

    async def go():
        async with _client(app) as c:
            body = {"model": "m", "system": "be brief", "messages": [{"role": "user", "content": "how many tokens is this?"}]}
            n = (await c.post("/v1/messages/count_tokens", json=body)).json()["input_tokens"]
            done = eng.counters["finished"]
            j = (await c.post("/v1/messages", json={**body, "max_tokens": 4})).json()
            assert n == j["usage"]["input_tokens"] + j["usage"]["cache_read_input_tokens"] and n > 10
            assert eng.counters["finished"] == done + 1                     # counting generated nothing
            bad = await c.post("/v1/messages/count_tokens", json={"model": "m", "messages": []})
            assert bad.status_code == 400 and bad.json()["type"] == "error"
    run(go())
