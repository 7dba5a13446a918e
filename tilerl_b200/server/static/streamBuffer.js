// Smooths bursty deltas into a steady reveal: text is queued and released on animation frames at a
// rate that adapts to the backlog (per frame at least backlog * dt / maxLagMs characters, so a burst
// shrinks by a factor e every `maxLagMs`; never slower than `baseCps`).
export class StreamBuffer {
  constructor(onText, {baseCps = 400, maxLagMs = 250, now = () => performance.now(),
                       raf = (cb) => requestAnimationFrame(cb)} = {}) {
    this.onText = onText; this.baseCps = baseCps; this.maxLagMs = maxLagMs; this.now = now; this.raf = raf;
    this.queue = ""; this.last = null; this.running = false; this.closed = false; this.onDrain = null;
  }
  push(text) { this.queue += text; if (!this.running) { this.running = true; this.last = this.now(); this.raf(() => this._tick()); } }
  end(onDrain) { this.closed = true; this.onDrain = onDrain; if (!this.running && onDrain) onDrain(); }
  flush() { if (this.queue) { this.onText(this.queue); this.queue = ""; } }
  _tick() {
    const t = this.now(), dt = Math.max(0, t - this.last); this.last = t;
    // rate needed to clear the backlog within maxLagMs, but at least the base rate
    const cps = Math.max(this.baseCps, this.queue.length * 1000 / this.maxLagMs);
    let n = Math.max(1, Math.floor(cps * dt / 1000));
    if (n >= this.queue.length) n = this.queue.length;
    if (n > 0) { this.onText(this.queue.slice(0, n)); this.queue = this.queue.slice(n); }
    if (this.queue.length) this.raf(() => this._tick());
    else { this.running = false; if (this.closed && this.onDrain) this.onDrain(); }
  }
}
