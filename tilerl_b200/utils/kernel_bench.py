"""Time individual kernels at the 27B's projection shapes with CUDA events.

    python -m tilerl_b200.utils.kernel_bench [--m 1] [--only gemm|gemv|quant|fp8] [--reps 20]
    python -m tilerl_b200.utils.kernel_bench --only attn --ctx 32768 --batch 1 [--splits 37] [--eager 5]

Each measurement rotates over enough distinct weight copies to exceed the 126 MB L2,
so every launch streams its weights from HBM; the figure printed is achieved weight
bytes per second of the launch (or launch pair) named.
"""
from __future__ import annotations

import argparse
import json

import torch

SHAPES = {"gate_up": (34816, 5120), "down": (5120, 17408), "gdn_in": (16480, 5120),
          "qkv": (14336, 5120), "o": (5120, 6144)}


def attention_bench(args):
    """One attention layer of the 27B at decode (prep + split-KV kernel + combine) over a paged pool
    holding ``--batch`` sequences of ``--ctx`` tokens: device time per layer and K / V bytes per second.
    ``--eager N`` runs N plain launches instead (the form to put under a profiler)."""
    from tilerl_b200.batch import Batch
    from tilerl_b200.config import get_config
    from tilerl_b200.factory import make_ops
    from tilerl_b200.kv import PagedKvPool
    dev = "cuda"
    cfg = get_config("qwen38-27b")
    ops = make_ops(dev)
    n_q, n_kv, d = cfg.n_q_heads, cfg.n_kv_heads, cfg.head_dim
    rows = n_q * 2 * d + 2 * n_kv * d
    lp = {"q_norm": torch.ones(d, device=dev), "k_norm": torch.ones(d, device=dev)}
    ctx, b = args.ctx, args.batch
    nb = (ctx + 16) // 16 + 1
    pool = PagedKvPool(cfg, b * nb + 2, dev, dtype=torch.bfloat16)
    kc, vc = pool.layer(0)
    kc.normal_()
    vc.normal_()
    seqs = [dict(tokens=[1], start=ctx, blocks=list(range(1 + i * nb, 1 + (i + 1) * nb)), slot=i + 1) for i in range(b)]
    batch = Batch.build(seqs, dev)
    qkv = (torch.randn(b, rows, device=dev) * 0.5).to(torch.bfloat16)
    out = []
    for splits in ([args.splits] if args.splits >= 0 else (0, 4, 9, 18, 37, 64)):
        ops.attn_splits = splits
        if args.eager:
            for _ in range(args.eager):
                ops.attention(qkv, lp, batch, pool, 0, cfg, n_q, n_kv)
            torch.cuda.synchronize()
            continue
        for _ in range(3):
            ops.attention(qkv, lp, batch, pool, 0, cfg, n_q, n_kv)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for _ in range(args.reps):
                ops.attention(qkv, lp, batch, pool, 0, cfg, n_q, n_kv)
        g.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        g.replay()
        e1.record()
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) / args.reps * 1e3
        kv_bytes = 2 * b * ctx * n_kv * d * 2
        out.append({"ctx": ctx, "batch": b, "splits": splits or "auto", "us_per_layer": round(us, 1),
                    "kv_MB": round(kv_bytes / 1e6), "TBps": round(kv_bytes / us / 1e6, 2)})
    print(json.dumps(out, indent=1))
    print("kernel_bench done")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--m", type=int, default=1)
    ap.add_argument("--terms", type=int, default=4)
    ap.add_argument("--only", default="")
    ap.add_argument("--reps", type=int, default=20)
    ap.add_argument("--shapes", default="")
    ap.add_argument("--max-ctas", type=int, default=0)
    ap.add_argument("--split", type=int, default=1)
    ap.add_argument("--tiled", type=int, default=1)
    ap.add_argument("--trace", action="store_true", help="gemm: per-phase timestamps of one launch (median, max over CTAs)")
    ap.add_argument("--ctx", type=int, default=32768, help="attn: context length")
    ap.add_argument("--batch", type=int, default=1, help="attn: sequences")
    ap.add_argument("--splits", type=int, default=-1, help="attn: KV splits (0 = the backend's choice, -1 = sweep)")
    ap.add_argument("--eager", type=int, default=0, help="attn: this many plain launches, no timing")
    args = ap.parse_args()
    if args.only == "attn":
        return attention_bench(args)
    from tilerl_b200.formats import NVFP4Tensor
    from tilerl_b200.ops.cuda import CudaOps
    from tilerl_b200.ops.gemm_tc import gemm_nvfp4, quant_act, sf_tiled, w_stream, wq_tiled
    from tilerl_b200.ops import native
    dev = torch.device("cuda", 0)
    ops = CudaOps(dev)
    ops.tile_weights = bool(args.tiled)
    out = {}
    names = [s for s in args.shapes.split(",") if s] or list(SHAPES)
    for name in names:
        n, k = SHAPES[name]
        wbytes = n * k // 2 + n * k // 16
        copies = max(2, int(400e6 // wbytes) + 1)
        ws = []
        for c in range(copies):
            w = NVFP4Tensor(torch.randint(0, 255, (n, k // 2), dtype=torch.uint8, device=dev),
                            (torch.rand(n, k // 16, device=dev) + 0.5).to(torch.float8_e4m3fn),
                            torch.ones(1, device=dev))
            sf_tiled(w)
            wq_tiled(w)
            w_stream(w)
            ws.append(w)
        x = torch.randn(args.m, k, device=dev).to(torch.bfloat16)
        y = torch.zeros(args.m, n, dtype=torch.bfloat16, device=dev)
        res = {}

        def timeit(fn):
            """Device time per launch: the launches are captured in one CUDA graph so the
            host launch path is not part of the figure."""
            for i in range(3):
                fn(ws[i % copies])
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                for i in range(args.reps):
                    fn(ws[i % copies])
            g.replay()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            g.replay()
            e1.record()
            torch.cuda.synchronize()
            return e0.elapsed_time(e1) / args.reps * 1e3  # us

        if args.only in ("", "gemv") and args.m <= 8:
            us = timeit(lambda w: ops.gemv_now(x, w, y))
            res["gemv_simt_us"] = round(us, 2)
            res["gemv_simt_TBs"] = round(wbytes / us / 1e6, 3)
        if args.only in ("", "gemm"):
            us = timeit(lambda w: gemm_nvfp4(ops, x, w, y, terms=args.terms, max_ctas=args.max_ctas, split=bool(args.split)))
            res["quant+gemm_tc_us"] = round(us, 2)
            res["quant+gemm_tc_TBs"] = round(wbytes / us / 1e6, 3)
            xq, sfx, rs = quant_act(ops, x, k, args.terms)
            from tilerl_b200.ops.gemm_tc import _scratch
            import ctypes
            ops.lib.trl_gemm_nvfp4_scratch_bytes.restype = ctypes.c_long
            nb = ops.lib.trl_gemm_nvfp4_scratch_bytes(args.m, args.terms, n, k, args.max_ctas)
            partial, counters = _scratch(ops, nb, 8192)

            def gemm_only(w):
                native.check(ops.lib.trl_gemm_nvfp4(
                    (w.wq_tiled if args.tiled else w.wq).data_ptr(), w.sf_tiled.data_ptr(), w.tscale.data_ptr(), xq.data_ptr(), sfx.data_ptr(),
                    rs.data_ptr(), None, 0, y.data_ptr(), y.stride(0), partial.data_ptr(), counters.data_ptr(),
                    partial.numel() * 4, args.m, args.terms, n, k, 0, args.max_ctas, args.split, args.tiled, native.stream()))
            us = timeit(gemm_only)
            res["gemm_tc_us"] = round(us, 2)
            res["gemm_tc_TBs"] = round(wbytes / us / 1e6, 3)
            if args.trace:
                # one traced launch: phase timestamps per CTA, reported in us after the first CTA's entry
                # needs the timeline build: python -m tilerl_b200.build --trace; TRL_TRACE_LIB=1
                import numpy as np
                gemm_only(ws[0])
                torch.cuda.synchronize()
                buf = np.zeros((148, 16), dtype=np.uint64)
                native.check(ops.lib.trl_gemm_trace_read(buf.ctypes.data, 148), "trace_read")
                t = buf.astype(np.float64)
                live = t[:, 0] > 0
                t0 = t[live, 0].min()
                names = ["entry", "setup", "dep_wait", "first_operands", "last_mma", "first_accum", "tmem_read",
                         "finish", "teardown", "seg_counted", "reduce_start", "reduce_batch0"]
                res["trace_us"] = {nm: [round(float(np.median(t[live, i] - t0)) / 1e3, 2),
                                        round(float((t[live, i] - t0).max()) / 1e3, 2)]
                                   for i, nm in enumerate(names)}
        if args.only == "fp8":
            # block-scaled FP8 weights of the same shape: quantiser + tcgen05 GEMM, or the GEMV up to 8 rows
            from tilerl_b200.formats import FP8BlockTensor
            from tilerl_b200.ops import gemm_fp8
            del ws
            torch.cuda.empty_cache()
            fbytes = n * k + (n // 128 + 1) * (k // 128) * 4
            ws = [FP8BlockTensor(torch.randint(0, 120, (n, k), dtype=torch.uint8, device=dev).view(torch.float8_e4m3fn),
                                 torch.rand((n + 127) // 128, k // 128, device=dev) + 0.5)
                  for _ in range(max(2, int(400e6 // fbytes) + 1))]
            copies = len(ws)
            if args.m <= gemm_fp8.GEMV_ROWS:
                us = timeit(lambda w: gemm_fp8.gemv(ops, x, w, y))
                res["gemv_fp8_us"] = round(us, 2)
                res["gemv_fp8_TBs"] = round(fbytes / us / 1e6, 3)
            us = timeit(lambda w: gemm_fp8.gemm(ops, x, w, y))
            res["quant+gemm_fp8_us"] = round(us, 2)
            res["quant+gemm_fp8_TFLOPs"] = round(2.0 * args.m * n * k / us / 1e6, 1)
            x8, sc = gemm_fp8.quant_act(ops, x)

            def fp8_only(w):
                native.check(ops.lib.trl_gemm_fp8(w.w8.data_ptr(), w.wscale.data_ptr(), x8.data_ptr(), sc.data_ptr(),
                                                  None, 0, y.data_ptr(), y.stride(0), args.m, n, k, 0, native.stream()))
            us = timeit(fp8_only)
            res["gemm_fp8_us"] = round(us, 2)
            res["gemm_fp8_TFLOPs"] = round(2.0 * args.m * n * k / us / 1e6, 1)
        if args.only in ("", "quant"):
            us = timeit(lambda w: quant_act(ops, x, k, args.terms))
            res["quant_us"] = round(us, 2)
        out[name] = res
        del ws
        torch.cuda.empty_cache()
    print(json.dumps(out, indent=1))
    print("kernel_bench done")


if __name__ == "__main__":
    main()
