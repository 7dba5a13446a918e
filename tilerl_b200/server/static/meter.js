// Time to first token and decode rate of the running answer, from the deltas seen by the client.
export class Meter {
  constructor(el, now = () => performance.now()) { this.el = el; this.now = now; this.reset(); }
  reset() { this.t0 = this.now(); this.first = null; this.chars = 0; this.el.textContent = ""; }
  onDelta(text) { if (this.first === null) this.first = this.now(); this.chars += text.length; this.show(); }
  onDone(usage) {
    const dt = (this.now() - (this.first ?? this.t0)) / 1000;
    const n = usage && usage.completion_tokens ? usage.completion_tokens : 0;
    this.el.textContent = `ttft ${((this.first ?? this.now()) - this.t0).toFixed(0)} ms` +
      (n && dt > 0 ? ` | ${(n / dt).toFixed(1)} tok/s | ${n} tokens` : "");
  }
  show() { this.el.textContent = `ttft ${(this.first - this.t0).toFixed(0)} ms | ${this.chars} chars`; }
}
