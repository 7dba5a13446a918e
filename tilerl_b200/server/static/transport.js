// One request per socket: open, send the request, deliver parsed frames, close.  A socket that drops
// before the final frame is reopened (at most `retries` times) with the SAME request: its
// idempotency_key makes the server join the run in flight or replay the finished answer, and the text
// already shown is skipped by counting characters per channel.
import {parseFrame} from "./protocol.js";

export function wsUrl(loc = window.location) {
  return (loc.protocol === "https:" ? "wss://" : "ws://") + loc.host + "/ws/chat";
}

export function startChat(request, handlers, url = wsUrl(), retries = 1, Socket = WebSocket) {
  let ws = null, finished = false, left = request.idempotency_key ? retries : 0;
  const shown = {reasoning: 0, content: 0};
  const finish = (f) => { if (!finished) { finished = true; handlers.onEnd && handlers.onEnd(f); } };
  const lost = (message) => {
    if (finished) return;
    if (left > 0) { left--; open(); } else finish({type: "error", message});
  };
  function open() {
    const seen = {reasoning: 0, content: 0};       // characters this socket has delivered so far
    ws = new Socket(url);
    const mine = ws;
    ws.onopen = () => mine.send(JSON.stringify(request));
    ws.onmessage = (ev) => {
      if (mine !== ws) return;
      const f = parseFrame(ev.data);
      if (f.type === "delta") {
        const from = seen[f.channel];
        seen[f.channel] += f.text.length;
        const skip = Math.max(0, shown[f.channel] - from);   // a joined run repeats the prefix: show only what is new
        if (skip < f.text.length) {
          shown[f.channel] += f.text.length - skip;
          handlers.onDelta && handlers.onDelta(f.channel, f.text.slice(skip));
        }
      } else if (f.type === "tool_calls") handlers.onToolCalls && handlers.onToolCalls(f.tool_calls);
      else { finish(f); mine.close(); }
    };
    ws.onerror = () => { if (mine === ws) lost("connection error"); };
    ws.onclose = () => { if (mine === ws) lost("connection closed before the answer was complete"); };
  }
  open();
  return {cancel() {            // the Stop button: tell the server to end the run, then close
    finished = true;
    try { if (ws.readyState === 1) ws.send(JSON.stringify({type: "cancel"})); } catch (e) { /* closing anyway */ }
    ws.close();
  }};
}
