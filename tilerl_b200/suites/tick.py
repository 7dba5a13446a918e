"""Run a few eager decode ticks (and optionally one prefill) of a model so a profiler
can list every kernel of a tick with its device time.

    python -m tilerl_b200.suites.tick --model qwen38-27b --ticks 3 --ctx 512

Under ``ncu --metrics gpu__time_duration.sum`` the last tick's launches give the
per-kernel time shares of the decode tick.  With ``--events`` the script prints its
own per-op CUDA-event breakdown instead (no profiler needed).
"""
from __future__ import annotations

import argparse
import collections
import json

import torch


def main(argv=None):
    ap = argparse.ArgumentParser(prog="tilerl_b200.suites.tick")
    ap.add_argument("--model", default="qwen38-27b")
    ap.add_argument("--ticks", type=int, default=3)
    ap.add_argument("--ctx", type=int, default=512)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--prefill", type=int, default=0, help="also run one prefill of this many tokens")
    ap.add_argument("--events", action="store_true")
    args = ap.parse_args(argv)
    from tilerl_b200.batch import Batch
    from tilerl_b200.config import get_config
    from tilerl_b200.factory import build_model, make_ops
    from tilerl_b200.kv import GdnStatePool, PagedKvPool
    dev = torch.device("cuda", 0)
    cfg = get_config(args.model)
    ops = make_ops(dev)
    model = build_model(cfg, dev, seed=0, ops=ops)
    nblk = (args.ctx + args.ticks + max(args.prefill, 1) + 32) // 16 + 1
    kv = PagedKvPool(cfg, args.batch * nblk + 2, dev)
    st = GdnStatePool(cfg, args.batch + 1, dev)
    rows = [dict(blocks=list(range(1 + r * nblk, 1 + (r + 1) * nblk)), slot=r + 1) for r in range(args.batch)]
    times = collections.defaultdict(float)
    if args.events:
        _wrap(ops, times)
    if args.prefill:
        seqs = [dict(tokens=[1] * args.prefill, start=0, **r) for r in rows]
        for _ in range(2):   # the second pass is warm (weights tiled, workspace allocated)
            times.clear()
            model.forward(Batch.build(seqs, dev), ops, kv, st)
            torch.cuda.synchronize()
        if args.events:
            print(json.dumps({"prefill_ms": dict(times)}))
            times.clear()
    for i in range(args.ticks):
        seqs = [dict(tokens=[5], start=args.ctx + i, **r) for r in rows]
        batch = Batch.build(seqs, dev)
        ops.attn_splits = 32 if args.batch == 1 else 0
        if args.events:
            times.clear()
        logits = model.forward(batch, ops, kv, st)
        ops.argmax(logits)
        torch.cuda.synchronize()
    if args.events:
        print(json.dumps({"tick_ms": {k: round(v, 4) for k, v in sorted(times.items(), key=lambda kv: -kv[1])},
                          "total_ms": round(sum(times.values()), 3)}))
    print("tick suite done")


def _wrap(ops, times):
    """Time every op-surface call with CUDA events (synchronising; for breakdowns only)."""
    for name in ("embed", "norm_linear", "norm_linear_swiglu", "linear_residual", "attention", "gdn", "lm_head"):
        fn = getattr(ops, name)

        def timed(*a, _fn=fn, _name=name, **k):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            e0.record()
            out = _fn(*a, **k)
            e1.record()
            torch.cuda.synchronize()
            shape = tuple(a[0].shape) if hasattr(a[0], "shape") else ()
            w = a[2] if _name in ("norm_linear", "norm_linear_swiglu") else (a[1] if _name == "linear_residual" else None)
            key = _name + (f"[{w.shape[0]}x{w.shape[1]}]" if w is not None and hasattr(w, "shape") else "")
            times[key] += e0.elapsed_time(e1)
            return out

        setattr(ops, name, timed)


if __name__ == "__main__":
    main()
