"""Contract between the static web client and the server's WebSocket endpoint, checked without a
JavaScript runtime: the frame types, delta channels and request keys are read out of the client's
modules as text and held against a recorded live session of ``/ws/chat`` (plain chat, reasoning,
tool call, error), and the client's reveal buffer is re-stated in Python and checked for the
properties its comments promise.

Parity: the reference tests its TypeScript client against recorded WebSocket fixtures
(web/test/*.test.ts); here the fixtures are produced by the server under test in the same run.
"""
import json
import os
import re
import time

import pytest

from helpers import make_engine
from tilerl_b200.config import tiny
from tilerl_b200.server.app import create_app
from tilerl_b200.tokenizer import ByteTokenizer

STATIC = os.path.join(os.path.dirname(__file__), "..", "tilerl_b200", "server", "static")


def _js(name):
    with open(os.path.join(STATIC, name)) as f:
        return f.read()


def _js_string_array(src, name):
    m = re.search(name + r"\s*=\s*\[([^\]]*)\]", src)
    assert m, name
    return re.findall(r'"([^"]+)"', m.group(1))


@pytest.fixture()
def served():
    eng = make_engine(tiny(max_ctx=2048), blocks=300, slots=6)
    tok = ByteTokenizer()
    eng.eos_id = tok.eos_id
    eng.detok = tok.decode
    eng.think_ids = tok.think_ids
    eng.run(batching_window_s=0.0)
    yield eng, create_app(eng, tok, "tiny-test")
    eng.stop()


def _session(app, request):
    from starlette.testclient import TestClient
    frames = []
    with TestClient(app) as tc:
        with tc.websocket_connect("/ws/chat") as ws:
            ws.send_text(json.dumps(request) if not isinstance(request, str) else request)
            while True:
                f = json.loads(ws.receive_text())
                frames.append(f)
                if f["type"] in ("done", "error"):
                    break
    return frames


def _check_frames(frames, frame_types):
    """The order the client's protocol module documents: deltas, at most one tool_calls, then exactly
    one done or error; every delta carries a string on a known channel."""
    kinds = [f["type"] for f in frames]
    assert set(kinds) <= set(frame_types), kinds
    assert kinds[-1] in ("done", "error") and kinds.count("done") + kinds.count("error") == 1
    assert kinds.count("tool_calls") <= 1
    body = kinds[:-1]
    if "tool_calls" in body:
        assert body.index("tool_calls") == len(body) - 1
    for f in frames:
        if f["type"] == "delta":
            assert isinstance(f["text"], str) and f["channel"] in ("reasoning", "content")
        if f["type"] == "done":
            u = f["usage"]
            assert u["total_tokens"] == u["prompt_tokens"] + u["completion_tokens"]
            assert isinstance(f["finish_reason"], str)
        if f["type"] == "error":
            assert isinstance(f["message"], str)
        if f["type"] == "tool_calls":
            for c in f["tool_calls"]:
                assert c["type"] == "function" and isinstance(c["function"]["name"], str)
                json.loads(c["function"]["arguments"])


def test_frames_of_live_sessions_follow_the_clients_protocol(served):
    eng, app = served
    proto = _js("protocol.js")
    frame_types = _js_string_array(proto, "FRAME_TYPES")
    assert frame_types == ["delta", "tool_calls", "done", "error"]
    sessions = {
        "plain": {"messages": [{"role": "user", "content": "hi"}], "max_tokens": 6},
        "thinking": {"messages": [{"role": "user", "content": "hi"}], "max_tokens": 12, "enable_thinking": True},
        "sampled": {"messages": [{"role": "user", "content": "hi"}], "max_tokens": 6, "temperature": 0.8, "top_p": 0.9,
                    "top_k": 5, "seed": 3},
        "malformed": "{not json",
        "no_messages": {"max_tokens": 4},
    }
    recorded = {}
    for name, req in sessions.items():
        frames = _session(app, req)
        _check_frames(frames, frame_types)
        recorded[name] = [f["type"] for f in frames]
    assert recorded["plain"][-1] == "done" and recorded["sampled"][-1] == "done"
    assert recorded["malformed"] == ["error"] and recorded["no_messages"] == ["error"]
    text = "".join(f["text"] for f in _session(app, sessions["plain"]) if f["type"] == "delta")
    assert isinstance(text, str)


def test_every_request_key_the_client_may_send_is_accepted(served):
    eng, app = served
    proto = _js("protocol.js")
    m = re.search(r"for \(const k of \[([^\]]*)\]\)", proto, re.S)
    assert m
    keys = re.findall(r'"([^"]+)"', m.group(1))
    assert {"max_tokens", "temperature", "top_p", "seed", "stop", "tools"} <= set(keys)
    values = {"max_tokens": 4, "temperature": 0.7, "top_p": 0.9, "top_k": 4, "seed": 1, "stop": ["\n\n"],
              "tools": [{"type": "function", "function": {"name": "f", "description": "d",
                                                          "parameters": {"type": "object", "properties": {}}}}],
              "enable_thinking": False, "reasoning_effort": "low", "idempotency_key": "turn-0123"}
    assert set(keys) <= set(values), set(keys) - set(values)
    for k in keys:                       # one key at a time, so a rejected key is named
        frames = _session(app, {"messages": [{"role": "user", "content": "hi"}], "stream": True, k: values[k],
                                **({} if k == "max_tokens" else {"max_tokens": 4})})
        assert frames[-1]["type"] == "done", (k, frames[-1])


def test_modules_import_only_each_other_and_touch_the_dom_only_in_render_and_main():
    mods = [f for f in os.listdir(STATIC) if f.endswith(".js")]
    for mod in mods:
        src = _js(mod)
        for target in re.findall(r'from\s+"([^"]+)"', src):
            assert target.startswith("./") and os.path.exists(os.path.join(STATIC, target[2:])), (mod, target)
        if mod not in ("render.js", "main.js", "meter.js"):
            assert "document." not in src, mod
    index = open(os.path.join(STATIC, "index.html")).read()
    assert 'type="module"' in index and "main.js" in index


class _PyStreamBuffer:
    """Line-by-line restatement of streamBuffer.js::StreamBuffer for a fake clock and frame queue."""

    def __init__(self, on_text, base_cps=400, max_lag_ms=250, now=None, raf=None):
        self.on_text, self.base_cps, self.max_lag_ms, self.now, self.raf = on_text, base_cps, max_lag_ms, now, raf
        self.queue, self.last, self.running, self.closed, self.on_drain = "", None, False, False, None

    def push(self, text):
        self.queue += text
        if not self.running:
            self.running, self.last = True, self.now()
            self.raf(self._tick)

    def end(self, on_drain):
        self.closed, self.on_drain = True, on_drain
        if not self.running and on_drain:
            on_drain()

    def _tick(self):
        t = self.now()
        dt = max(0, t - self.last)
        self.last = t
        cps = max(self.base_cps, len(self.queue) * 1000 / self.max_lag_ms)
        n = max(1, int(cps * dt / 1000))
        n = min(n, len(self.queue))
        if n > 0:
            self.on_text(self.queue[:n])
            self.queue = self.queue[n:]
        if self.queue:
            self.raf(self._tick)
        else:
            self.running = False
            if self.closed and self.on_drain:
                self.on_drain()


def test_reveal_buffer_keeps_order_and_bounds_the_lag():
    src = _js("streamBuffer.js")
    # the restatement follows the module's constants and formula
    assert "baseCps = 400" in src and "maxLagMs = 250" in src
    assert "this.queue.length * 1000 / this.maxLagMs" in src
    clock = [0.0]
    frames = []
    out = []
    shown_at = []
    buf = _PyStreamBuffer(lambda s: (out.append(s), shown_at.append(clock[0])), now=lambda: clock[0],
                          raf=frames.append)
    drained = []
    burst = "x" * 5000                       # a burst far above the base rate
    buf.push("hello ")
    buf.push(burst)
    buf.end(lambda: drained.append(clock[0]))
    backlog = []
    while frames:                            # 60 Hz animation frames
        clock[0] += 1000 / 60
        frames.pop(0)()
        backlog.append((clock[0], len(buf.queue)))
    assert "".join(out) == "hello " + burst                 # nothing lost, nothing reordered
    # the backlog shrinks at least by the factor (1 - dt / maxLag) per frame: e-fold every 250 ms
    total = len("hello " + burst)
    for t, left in backlog:
        k = round(t / (1000 / 60))           # frames so far; the floor in the module costs at most one character each
        assert left <= total * (1 - (1000 / 60) / 250) ** k + k + 1, (t, left)
    assert drained and drained[0] <= 8 * 250                  # 5000 characters gone within 2 s
    assert len(out) > 5                                      # revealed over several frames, not at once


def test_a_retried_turn_joins_or_replays_and_a_cancel_frame_stops_the_run(served):
    eng, app = served
    req = {"messages": [{"role": "user", "content": "go on"}], "stream": True, "max_tokens": 6, "temperature": 1.0,
           "idempotency_key": "turn-abc"}
    first = _session(app, req)
    done = eng.counters["finished"]
    second = _session(app, req)                               # the retry: same key, nothing generated
    text = lambda frames: "".join(f["text"] for f in frames if f["type"] == "delta")
    assert first[-1]["type"] == second[-1]["type"] == "done" and text(first) == text(second)
    assert first[-1]["usage"] == second[-1]["usage"] and eng.counters["finished"] == done
    # the Stop button: a cancel frame ends a keyed run for good, and the key is free again
    from starlette.testclient import TestClient
    slow = {**req, "idempotency_key": "turn-stop", "max_tokens": 1500}
    with TestClient(app) as tc:
        with tc.websocket_connect("/ws/chat") as ws:
            ws.send_text(json.dumps(slow))
            ws.send_text(json.dumps({"type": "cancel"}))
            frames = []
            while True:
                f = json.loads(ws.receive_text())
                frames.append(f)
                if f["type"] in ("done", "error"):
                    break
    assert frames[-1] == {"type": "error", "message": "cancelled", "code": "cancelled"} or frames[-1]["type"] == "done"
    if frames[-1]["type"] == "error":       # (cancelled in flight, or already finished and discarded unsent)
        assert app.state.ctx.keys.lookup("turn-stop") is None
    for _ in range(200):
        if eng.kv.used_blocks == 0:
            break
        time.sleep(0.01)
    assert eng.kv.used_blocks == 0


def _replay_skip(shown, sockets):
    """transport.js: per channel, a socket counts what it has delivered (`seen`); text below the count already
    shown by earlier sockets (`shown`) is skipped."""
    out = ""
    for deltas in sockets:
        seen = 0
        for t in deltas:
            start, seen = seen, seen + len(t)
            skip = max(0, shown - start)
            if skip < len(t):
                shown += len(t) - skip
                out += t[skip:]
    return out


def test_transport_shows_each_character_once_when_a_socket_is_reopened():
    src = _js("transport.js")
    assert "Math.max(0, shown[f.channel] - from)" in src and "f.text.slice(skip)" in src
    assert 'JSON.stringify({type: "cancel"})' in src and "request.idempotency_key ? retries : 0" in src
    answer = "the quick brown fox jumps over the lazy dog"
    # the first socket dies after 17 characters; the second replays the answer in other pieces
    assert _replay_skip(0, [["the qu", "ick brown f"], ["the quick ", "brown fox jum", "ps over the lazy dog"]]) == answer
    assert _replay_skip(0, [[answer], [answer]]) == answer              # dropped after everything but the final frame
    assert _replay_skip(0, [[], ["the quick", answer[9:]]]) == answer   # dropped before the first delta
    key = _js("protocol.js")
    assert "export function newKey" in key and '"turn-" + s' in key
