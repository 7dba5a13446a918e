// Minimal safe renderer: escapes HTML, then fenced code blocks, inline code, bold, links and
// paragraphs.  Reasoning text goes in a collapsible block above the answer.
const ESC = {"&": "&amp;", "<": "&lt;", ">": "&gt;", '"': "&quot;", "'": "&#39;"};
export const escapeHtml = (s) => s.replace(/[&<>"']/g, (c) => ESC[c]);

export function renderMarkdown(src) {
  const parts = src.split(/```/);
  let html = "";
  for (let i = 0; i < parts.length; i++) {
    if (i % 2 === 1) {                       // inside a fence (an unterminated fence renders as code too)
      const nl = parts[i].indexOf("\n");
      const lang = nl >= 0 ? parts[i].slice(0, nl).trim() : "";
      const body = nl >= 0 ? parts[i].slice(nl + 1) : parts[i];
      html += `<pre><code${lang ? ` data-lang="${escapeHtml(lang)}"` : ""}>${escapeHtml(body)}</code></pre>`;
    } else {
      let t = escapeHtml(parts[i]);
      t = t.replace(/`([^`\n]+)`/g, "<code>$1</code>");
      t = t.replace(/\*\*([^*\n]+)\*\*/g, "<b>$1</b>");
      t = t.replace(/\[([^\]\n]+)\]\((https?:\/\/[^\s)]+)\)/g, '<a href="$2" target="_blank" rel="noopener">$1</a>');
      html += t.split(/\n{2,}/).map((p) => p.trim() ? `<p>${p.replace(/\n/g, "<br>")}</p>` : "").join("");
    }
  }
  return html;
}

export class MessageView {
  constructor(root, role) {
    this.el = document.createElement("div"); this.el.className = "msg " + role;
    this.think = document.createElement("details"); this.think.className = "think"; this.think.hidden = true;
    this.think.innerHTML = "<summary>reasoning</summary><div class='body'></div>";
    this.body = document.createElement("div"); this.body.className = "body";
    this.tools = document.createElement("div"); this.tools.className = "tools";
    this.el.append(this.think, this.body, this.tools); root.append(this.el);
    this.text = {reasoning: "", content: ""};
  }
  append(channel, text) {
    this.text[channel] += text;
    if (channel === "reasoning") { this.think.hidden = false; this.think.querySelector(".body").textContent = this.text.reasoning; }
    else this.body.innerHTML = renderMarkdown(this.text.content);
    this.el.scrollIntoView({block: "end"});
  }
  toolCalls(calls) {
    this.tools.innerHTML = calls.map((c) => `<div class="tool"><b>${escapeHtml(c.function.name)}</b>` +
      `<pre>${escapeHtml(c.function.arguments)}</pre></div>`).join("");
  }
  fail(message) { const e = document.createElement("div"); e.className = "error"; e.textContent = message; this.el.append(e); }
}
