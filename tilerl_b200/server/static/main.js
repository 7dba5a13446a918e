import {buildRequest, newKey} from "./protocol.js";
import {startChat} from "./transport.js";
import {StreamBuffer} from "./streamBuffer.js";
import {MessageView} from "./render.js";
import {Meter} from "./meter.js";

const log = document.getElementById("log"), form = document.getElementById("form"), input = document.getElementById("input");
const stopBtn = document.getElementById("stop"), meter = new Meter(document.getElementById("meter"));
const history = [];
let running = null;

function opts() {
  const v = (id) => document.getElementById(id).value;
  return {max_tokens: parseInt(v("max_tokens")) || 512, temperature: v("temperature") === "" ? undefined : parseFloat(v("temperature")),
          enable_thinking: document.getElementById("thinking").checked};
}

form.addEventListener("submit", (ev) => {
  ev.preventDefault();
  const text = input.value.trim();
  if (!text || running) return;
  input.value = "";
  history.push({role: "user", content: text});
  new MessageView(log, "user").append("content", text);
  const view = new MessageView(log, "assistant");
  const bufs = {reasoning: new StreamBuffer((t) => view.append("reasoning", t)), content: new StreamBuffer((t) => view.append("content", t))};
  meter.reset(); stopBtn.disabled = false;
  running = startChat(buildRequest(history, {...opts(), idempotency_key: newKey()}), {
    onDelta(ch, t) { meter.onDelta(t); bufs[ch].push(t); },
    onToolCalls(calls) { view.toolCalls(calls); },
    onEnd(f) {
      const finish = () => {
        if (f.type === "done") { history.push({role: "assistant", content: view.text.content}); meter.onDone(f.usage); }
        else view.fail(f.message || "error");
        running = null; stopBtn.disabled = true; input.focus();
      };
      bufs.reasoning.end(); bufs.content.end(finish);
    },
  });
});
stopBtn.addEventListener("click", () => { if (running) { running.cancel(); running = null; stopBtn.disabled = true; } });
input.addEventListener("keydown", (ev) => { if (ev.key === "Enter" && !ev.shiftKey) { ev.preventDefault(); form.requestSubmit(); } });
