"""Timings of the speculative-decode and long-context sparse-KV configurations on one GPU.

    python -m tilerl_b200.suites.serve --what spec   [--prompts 8 --gen 128 --width 8]
    python -m tilerl_b200.suites.serve --what sparse [--ctx 32768 --top-k 128 --ticks 32]
    python -m tilerl_b200.suites.serve --what batch  [--requests 8 --prompt-len 7400 --gen 256]

``spec``: B = 1, prompts of 80..300 random ids, a width-W verify tick timed at forced full
acceptance (drafts = the trunk's own greedy continuation), at zero acceptance (a constant
draft) and with the random-init block drafter, against plain decoding (``--graph 0``: eager verify ticks).
``batch``: ``--requests`` concurrent long prompts through continuous batching (chunked prefill,
then CUDA-graph decode ticks of the whole batch): prefill tok/s and aggregate decode tok/s.
``sparse``: one sequence prefilled to ``ctx`` tokens, then decode ticks with dense attention
(CUDA-graph) and with top-k page selection (Quest bounds, trailing window of 8 pages, refreshed
every 8 ticks).  All times are wall clock around device-synchronised loops.
"""
from __future__ import annotations

import argparse
import json
import time

import torch


def _sync_time(fn):
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    out = fn()
    torch.cuda.synchronize()
    return out, time.perf_counter() - t0


def spec(args, cfg, ops, model):
    from tilerl_b200.engine import SamplingParams
    from tilerl_b200.factory import build_engine
    from tilerl_b200.spec import BlockDrafter, BlockDrafterConfig, ConstantDrafter, OracleDrafter
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, cfg.vocab, (int(torch.randint(80, 301, (1,), generator=g)),), generator=g).tolist()
               for _ in range(args.prompts)]
    sp = SamplingParams(max_tokens=args.gen)
    out = {}
    plain = build_engine(model, ops, slots=2, max_ctx=1024, graph=True, prefix=False)
    plain.generate(prompts[:1], SamplingParams(max_tokens=8))
    conts = {}

    def run_plain():
        n = 0
        for p in prompts:
            r = plain.generate([p], sp)[0]
            conts[tuple(p)] = r.tokens
            n += len(r.tokens)
        return n
    n, dt = _sync_time(run_plain)
    out["plain"] = dict(tok_s=round(n / dt, 1), ticks=plain.counters["decode_ticks"])
    drafters = {"forced_full_acceptance": ConstantDrafter(1), "oracle_replay": OracleDrafter(conts),
                "zero_acceptance": ConstantDrafter(0),
                "block_drafter_random_init": BlockDrafter(model, BlockDrafterConfig(width=args.width), dtype=torch.bfloat16)}
    for name, d in drafters.items():
        eng = build_engine(model, ops, slots=2, max_ctx=1024, graph=bool(args.graph), prefix=False, spec_width=args.width,
                           drafter=d)
        eng.spec_force_accept = name == "forced_full_acceptance"
        eng.generate(prompts[:1], SamplingParams(max_tokens=8))
        c0 = dict(eng.counters)

        def run():
            return sum(len(eng.generate([p], sp)[0].tokens) for p in prompts)
        n, dt = _sync_time(run)
        ticks = eng.counters["decode_ticks"] - c0["decode_ticks"]
        drafted = eng.counters["spec_drafted"] - c0["spec_drafted"]
        acc = eng.counters["spec_accepted"] - c0["spec_accepted"]
        out[name] = dict(tok_s=round(n / dt, 1), verify_ticks=ticks, ms_per_verify_tick=round(1000 * dt / max(1, ticks), 2),
                         tokens_per_tick=round(n / max(1, ticks), 2), acceptance=round(acc / max(1, drafted), 3))
    return out


def sparse(args, cfg, ops, model):
    from tilerl_b200.engine import SamplingParams, StepLimits
    from tilerl_b200.factory import build_engine
    from tilerl_b200.sparse import SparseConfig, SparseKV
    g = torch.Generator().manual_seed(1)
    prompt = torch.randint(0, cfg.vocab, (args.ctx,), generator=g).tolist()
    out = {"ctx": args.ctx, "top_k_pages": args.top_k}
    for name in ("dense_graph", "sparse_eager"):
        skv = SparseKV(cfg, SparseConfig(top_k=args.top_k, window=8, refresh_ticks=8, min_tokens=4096)) \
            if name == "sparse_eager" else None
        eng = build_engine(model, ops, slots=2, max_ctx=args.ctx + 256, graph=skv is None, prefix=False, sparse=skv,
                           limits=StepLimits(max_batched_tokens=2048))
        rid = eng.submit(prompt, SamplingParams(max_tokens=args.ticks + 8, ignore_eos=True))
        def prefill():
            while eng.poll(rid)["state"] not in ("decode", "done"):
                eng.step()
        _, t_pre = _sync_time(prefill)
        for _ in range(8):
            eng.step()
        _, dt = _sync_time(lambda: [eng.step() for _ in range(args.ticks)])
        out[name] = dict(prefill_s=round(t_pre, 2), prefill_tok_s=round(args.ctx / t_pre, 1),
                         ms_per_tick=round(1000 * dt / args.ticks, 2))
        if skv is not None:
            out[name]["stats"] = dict(skv.stats)
        eng.cancel(rid)
        del eng
        torch.cuda.empty_cache()
    return out


def batch(args, cfg, ops, model):
    """Continuous batching of ``--requests`` long prompts (uniform-random ids), greedy decode."""
    from tilerl_b200.engine import SamplingParams, StepLimits
    from tilerl_b200.factory import build_engine
    g = torch.Generator().manual_seed(2)
    prompts = [torch.randint(0, cfg.vocab, (args.prompt_len,), generator=g).tolist() for _ in range(args.requests)]
    eng = build_engine(model, ops, slots=args.requests + 1, max_ctx=args.prompt_len + args.gen + 64, graph=True,
                       prefix=False, limits=StepLimits(max_batch=args.requests, max_batched_tokens=2048),
                       kv_fp8=args.kv_format == "fp8")
    eng.generate([prompts[0][:64]], SamplingParams(max_tokens=4))
    eng.precapture((args.requests,))
    rids = [eng.submit(p, SamplingParams(max_tokens=args.gen, ignore_eos=True, temperature=args.temperature,
                                         top_p=args.top_p, top_k=args.sample_top_k, seed=i))
            for i, p in enumerate(prompts)]

    def prefill():
        while any(eng.poll(r)["state"] in ("waiting", "prefill") for r in rids):
            eng.step()
    _, t_pre = _sync_time(prefill)
    n0 = sum(eng.poll(r)["n_out"] for r in rids)
    ticks0 = eng.counters["decode_ticks"]

    def decode():
        while any(eng.poll(r)["state"] != "done" for r in rids):
            eng.step()
    _, t_dec = _sync_time(decode)
    n1 = sum(len(eng.take(r).tokens) for r in rids)
    ticks = eng.counters["decode_ticks"] - ticks0
    return dict(requests=args.requests, prompt_len=args.prompt_len, gen=args.gen, kv_format=args.kv_format,
                sampling=dict(temperature=args.temperature, top_p=args.top_p, top_k=args.sample_top_k),
                kv_pool_gib=round(2 * eng.kv.k.numel() * eng.kv.k.element_size() / 2 ** 30, 2),
                prefill_s=round(t_pre, 2), prefill_tok_s=round(args.requests * args.prompt_len / t_pre, 1),
                decode_s=round(t_dec, 2), decode_agg_tok_s=round((n1 - n0) / t_dec, 1),
                ms_per_decode_tick=round(1000 * t_dec / max(1, ticks), 2), graph_ticks=eng.counters["graph_ticks"])


def main(argv=None):
    ap = argparse.ArgumentParser(prog="tilerl_b200.suites.serve")
    ap.add_argument("--what", default="spec", choices=["spec", "sparse", "batch"])
    ap.add_argument("--requests", type=int, default=8)
    ap.add_argument("--prompt-len", type=int, default=7400)
    ap.add_argument("--model", default="qwen38-27b")
    ap.add_argument("--prompts", type=int, default=8)
    ap.add_argument("--gen", type=int, default=128)
    ap.add_argument("--width", type=int, default=8)
    ap.add_argument("--ctx", type=int, default=32768)
    ap.add_argument("--top-k", type=int, default=128)
    ap.add_argument("--ticks", type=int, default=32)
    ap.add_argument("--temperature", type=float, default=0.0, help="batch: sampling temperature (0 = greedy)")
    ap.add_argument("--top-p", type=float, default=1.0, help="batch: nucleus bound")
    ap.add_argument("--sample-top-k", type=int, default=0, help="batch: top-k restriction of the sampler")
    ap.add_argument("--kv-format", default="bf16", choices=["bf16", "fp8"], help="batch: KV pool format")
    ap.add_argument("--graph", type=int, default=1, help="spec: replay verify ticks from CUDA graphs")
    args = ap.parse_args(argv)
    from tilerl_b200.config import get_config
    from tilerl_b200.factory import build_model, make_ops
    cfg = get_config(args.model)
    ops = make_ops("cuda")
    model = build_model(cfg, "cuda", seed=0, ops=ops)
    res = {"spec": spec, "sparse": sparse, "batch": batch}[args.what](args, cfg, ops, model)
    print(json.dumps({"config": args.what, "model": cfg.name, **res}))


if __name__ == "__main__":
    main()
