// One request per socket: open, send the request, deliver parsed frames, close.
import {parseFrame} from "./protocol.js";

export function wsUrl(loc = window.location) {
  return (loc.protocol === "https:" ? "wss://" : "ws://") + loc.host + "/ws/chat";
}

export function startChat(request, handlers, url = wsUrl()) {
  const ws = new WebSocket(url);
  let finished = false;
  const finish = (f) => { if (!finished) { finished = true; handlers.onEnd && handlers.onEnd(f); } };
  ws.onopen = () => ws.send(JSON.stringify(request));
  ws.onmessage = (ev) => {
    const f = parseFrame(ev.data);
    if (f.type === "delta") handlers.onDelta && handlers.onDelta(f.channel, f.text);
    else if (f.type === "tool_calls") handlers.onToolCalls && handlers.onToolCalls(f.tool_calls);
    else { finish(f); ws.close(); }
  };
  ws.onerror = () => finish({type: "error", message: "connection error"});
  ws.onclose = () => finish({type: "error", message: "connection closed before the answer was complete"});
  return {cancel() { finished = true; ws.close(); }};   // closing the socket cancels the request server-side
}
