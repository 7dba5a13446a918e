// Wire contract of WS /ws/chat.  Client -> server: ONE JSON request (same body as
// POST /v1/chat/completions), then optionally {type:"cancel"} to stop the run for good; a socket that
// just drops leaves a request that carries an idempotency_key running, and the same request sent again
// with that key joins it (or replays its answer) instead of generating twice.
// Server -> client frames, in order:
//   {type:"delta", channel:"reasoning"|"content", text}   zero or more
//   {type:"tool_calls", tool_calls:[{id,type:"function",function:{name,arguments}}]}   at most one
//   {type:"done", finish_reason, usage:{prompt_tokens,completion_tokens,total_tokens}}  exactly one, or
//   {type:"error", message, code?}                                                      instead of done
export const FRAME_TYPES = ["delta", "tool_calls", "done", "error"];

export function parseFrame(text) {
  let f;
  try { f = JSON.parse(text); } catch (e) { return {type: "error", message: "bad frame: " + e.message}; }
  if (!f || !FRAME_TYPES.includes(f.type)) return {type: "error", message: "unknown frame type " + (f && f.type)};
  if (f.type === "delta") {
    if (typeof f.text !== "string") return {type: "error", message: "delta without text"};
    if (f.channel !== "reasoning" && f.channel !== "content") f.channel = "content";
  }
  if (f.type === "done" && !f.usage) f.usage = {prompt_tokens: 0, completion_tokens: 0, total_tokens: 0};
  return f;
}

export function buildRequest(messages, opts = {}) {
  const req = {messages, stream: true};
  for (const k of ["max_tokens", "temperature", "top_p", "top_k", "seed", "stop", "tools", "enable_thinking",
                   "reasoning_effort", "idempotency_key"]) if (opts[k] !== undefined && opts[k] !== null && opts[k] !== "") req[k] = opts[k];
  return req;
}

// One key per user submission: a retry of the same turn reuses it, a newly typed message gets a new one.
export function newKey(rand = Math.random) {
  let s = "";
  for (let i = 0; i < 32; i++) s += Math.floor(rand() * 16).toString(16);
  return "turn-" + s;
}
