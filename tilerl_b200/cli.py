"""Command line: ``python -m tilerl_b200.cli {serve,train,bench,generate,merge,ledger}``.

Parity: reference ``src/tilerl/cli.py`` -- ``cmd_serve:145``, ``_build_parser:507-1255``
(same verbs; one ``TRL_*`` environment namespace instead of the reference's ``TILERL_*``).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from typing import List, Optional


def _add_model_flags(p: argparse.ArgumentParser) -> None:
    p.add_argument("--model", default="tiny", help="model config name (see tilerl_b200.config)")
    p.add_argument("--checkpoint", default=None, help="HF-style checkpoint directory")
    p.add_argument("--tokenizer", default=None, help="tokenizer.json (default: byte tokenizer)")
    p.add_argument("--device", default=None, help="cuda | cpu (default: cuda when available)")
    p.add_argument("--seed", type=int, default=0)


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="tilerl_b200")
    sub = ap.add_subparsers(dest="cmd", required=True)

    s = sub.add_parser("serve", help="OpenAI / Anthropic compatible HTTP server")
    _add_model_flags(s)
    s.add_argument("--host", default="127.0.0.1")
    s.add_argument("--port", type=int, default=8000)
    s.add_argument("--slots", type=int, default=8)
    s.add_argument("--blocks", type=int, default=None)
    s.add_argument("--max-ctx", type=int, default=4096)
    s.add_argument("--max-batch", type=int, default=64)
    s.add_argument("--max-batched-tokens", type=int, default=512)
    s.add_argument("--max-inflight", type=int, default=1024)
    s.add_argument("--decode-graph", dest="graph", action="store_true", default=True)
    s.add_argument("--no-decode-graph", dest="graph", action="store_false")
    s.add_argument("--no-prefix", action="store_true")
    s.add_argument("--draft", default=None, choices=[None, "block", "chain"])
    s.add_argument("--draft-checkpoint", default=None, help="directory written by spec.save_drafter (kind is read from it)")
    s.add_argument("--spec-width", type=int, default=8)
    s.add_argument("--draft-attn-window-tokens", type=int, default=None,
                   help="trailing context rows the block drafter reads (omitted: $TRL_DRAFT_ATTN_WINDOW_TOKENS, else the "
                        "drafter's own setting)")
    s.add_argument("--sparse-k", type=int, default=0)
    s.add_argument("--scorer", default="quest", choices=["quest", "learned"],
                   help="sparse page scores: Quest min/max bounds, or the learned indexer")
    s.add_argument("--indexer", default=None, help="directory holding indexer.safetensors (for --scorer learned)")
    s.add_argument("--sparse-min-tokens", type=int, default=4096)
    s.add_argument("--sparse-window-tokens", type=int, default=128)
    s.add_argument("--state-bytes", type=int, default=0,
                   help="device budget in bytes for the prefix store's GDN snapshots (0: a share of what the KV pool leaves)")
    s.add_argument("--device-free", type=int, default=None, metavar="BYTES",
                   help="with --dry-run: plan against this many free device bytes instead of a whole B200")
    s.add_argument("--json", action="store_true", help="with --dry-run: print the memory rows as JSON")
    s.add_argument("--record-residency", action="store_true",
                   help="after building and warming the engine, append its resident peak and the static / transient split "
                        "to the bench store (with --port 0: record and exit)")
    s.add_argument("--sparse-prefill-tokens", type=int, default=0,
                   help="prefill tokens per tick of a fill of --sparse-min-tokens or more while other requests share "
                        "the engine (0: the whole --max-batched-tokens budget)")
    s.add_argument("--sparse-refresh-ticks", type=int, default=8)
    s.add_argument("--kv-format", default="bf16", choices=["bf16", "fp8"],
                   help="KV pool format: bf16, or e4m3 with one fp32 scale per token and head")
    s.add_argument("--kv-fp8", dest="kv_format", action="store_const", const="fp8", help="same as --kv-format fp8")
    s.add_argument("--device-reserve-mib", type=int, default=0,
                   help="device memory left out of the KV pool sizing (other tenants of the GPU, fragmentation)")
    s.add_argument("--kv-store", default=None, help="directory of the cold-start KV store")
    s.add_argument("--kv-cold-bytes", type=int, default=0, help="pinned host bytes for demoted prefix pages (0: off)")
    s.add_argument("--dram-bytes", type=int, default=1 << 30, help="host bytes for demoted GDN snapshots")
    s.add_argument("--cold-ssd-path", default=None, help="spill file behind the host tier")
    s.add_argument("--cold-ssd-bytes", type=int, default=0, metavar="BYTES",
                   help="capacity of the spill file (0 with --cold-ssd-path: half of the free space of its filesystem)")
    s.add_argument("--completion-timeout-s", type=float, default=600.0)
    s.add_argument("--stream-pace", action="store_true")
    s.add_argument("--stream-pace-depth", type=int, default=0, metavar="N",
                   help="tokens buffered before a paced stream starts (headroom for one stall of the engine)")
    s.add_argument("--no-warmup", action="store_true")
    s.add_argument("--dry-run", action="store_true", help="print the memory ledger and exit")
    s.add_argument("--no-card-guard", action="store_true", help="start even if other processes hold the GPU")

    t = sub.add_parser("train", help="SFT / GRPO / on-policy distillation")
    _add_model_flags(t)
    t.add_argument("--recipe", default=None)
    t.add_argument("--rl", action="store_true")
    t.add_argument("--opd", action="store_true")
    t.add_argument("--steps", type=int, default=None)
    t.add_argument("--group", type=int, default=None)
    t.add_argument("--prompts-per-step", type=int, default=None)
    t.add_argument("--max-tokens", type=int, default=None)
    t.add_argument("--micro", type=int, default=None)
    t.add_argument("--lora-rank", type=int, default=None)
    t.add_argument("--lr", type=float, default=None)
    t.add_argument("--optim", default=None, choices=[None, "adamw", "adafactor", "iso"])
    t.add_argument("--reward", default=None)
    t.add_argument("--clip-eps", type=float, default=0.2)
    t.add_argument("--kl-coef", type=float, default=0.0)
    t.add_argument("--prompts", default=None, help="jsonl of prompts (default: random token prompts)")
    t.add_argument("--prompt-len", type=int, default=16)
    t.add_argument("--save-model", default=None)
    t.add_argument("--load-adapter", default=None)
    t.add_argument("--served-fp4", action="store_true")
    t.add_argument("--deterministic", action="store_true",
                   help="deterministic torch algorithms and fixed seeds (repeatable runs, slower)")
    t.add_argument("--indexer-warmup", action="store_true", help="train the learned sparse-KV page indexer")
    t.add_argument("--ctx", type=int, default=None, help="sequence length of the indexer warm-up batches")
    t.add_argument("--eval-every", type=int, default=0, help="adapter runs: eval reward on held-out prompts every N steps")
    t.add_argument("--patience", type=int, default=3, help="adapter runs: stop after this many evals without improvement")
    t.add_argument("--runs", default=None, help="run manifest directory (default: $TRL_RUNS or ./runs)")
    t.add_argument("--data", default=None,
                   help="JSONL of {prompt, answer}: real prompts; the reward is an exact match of the completion's last number")
    t.add_argument("--eval-gsm8k", default=None,
                   help="JSONL of {prompt | question, answer}: greedy exact-match accuracy before and after the run")
    t.add_argument("--eval-n", type=int, default=100, help="rows of --eval-gsm8k to score")
    t.add_argument("--eval-max-new-tokens", type=int, default=256)
    t.add_argument("--length-penalty", type=float, default=0.0,
                   help="RL reward subtracts this per generated token: orders an all-right group by length (a group whose "
                        "task reward ties still gets no gradient from length alone)")
    t.add_argument("--lineage", default=None, metavar="ID", help="id of the run this one descends from")
    t.add_argument("--judge", action="store_true",
                   help="RL: let the policy order the rollouts of a group whose rule-based rewards tie (the rule decides first)")
    t.add_argument("--indexer-corpus", default=None, metavar="DIR",
                   help="--indexer-warmup over prepared spans: files {train,held}_<label>.jsonl of {ctx, ids} rows; reports "
                        "recall at --k-pages per held length before and after")
    t.add_argument("--indexer-control-corpus", default=None, metavar="DIR",
                   help="held spans of another corpus, scored before / after under the same trained weights")
    t.add_argument("--indexer-di", type=int, default=128, help="width of an indexer head")
    t.add_argument("--k-pages", type=int, default=128, help="pages the recall keeps")
    t.add_argument("--q-samples", type=int, default=16, help="query positions per span and layer")
    t.add_argument("--q-min-pos", type=int, default=0, help="query positions start here")
    t.add_argument("--held-spans", type=int, default=0, help="use this many held spans, dealt evenly over the lengths (0: all)")
    t.add_argument("--recall-threshold", type=float, default=0.0, help="gate: the worst after-recall must reach this")
    t.add_argument("--eval-mmlu", default=None, metavar="JSONL",
                   help="rows {question, choices[4], answer letter}: multiple-choice accuracy before and after")
    t.add_argument("--eval-curve-n", type=int, default=100,
                   help="rows of --eval-gsm8k scored every --eval-every steps (a fixed-seed subset)")
    t.add_argument("--eval-curve-seed", type=int, default=0)
    t.add_argument("--curve-target-pt", type=float, default=5.0,
                   help="effect in points the curve is there to locate; the run refuses when 50/sqrt(--eval-curve-n) exceeds it")
    t.add_argument("--max-think-tokens", type=int, default=0,
                   help="RL rollouts: cap on the reasoning span, closed by force past it (0: no cap)")
    t.add_argument("--allow-short-rollouts", action="store_true",
                   help="skip the rollout-length guards (before training and every five steps); smoke recipes want "
                        "the truncation, a real run almost never does")
    t.add_argument("--force", action="store_true", help="train again even if a run with these inputs already finished")
    t.add_argument("--json", action="store_true", help="print the run manifest as JSON instead of step lines")
    t.add_argument("--dry-run", action="store_true", help="print the training-side memory plan and exit")
    t.add_argument("--train-seq-len", type=int, default=0, metavar="S",
                   help="--dry-run: token rows per micro-batch of the checkpointed tape (default: prompt + --max-tokens)")
    t.add_argument("--zero", type=int, default=1, help="--dry-run: ranks a full-parameter run shards its state over (ZeRO-3)")

    b = sub.add_parser("bench", help="prefill / decode throughput, kernel roofline table, calibration")
    _add_model_flags(b)
    b.add_argument("--prompt-len", type=int, default=512)
    b.add_argument("--gen", type=int, default=64)
    b.add_argument("--batches", default="1")
    b.add_argument("--kernels", action="store_true", help="print the declared cost table and bounds")
    b.add_argument("--context", type=int, default=None, help="--kernels: pooled context tokens a decode tick reads (default: --prompt-len)")
    b.add_argument("--prefill", type=int, default=0, metavar="S", help="--kernels: print the prefill table for S tokens instead of decode")
    b.add_argument("--device-name", default=None,
                   help="--kernels: the part whose floors divide the table (default: this B200's measured floors; h20, h100, v100: nominal)")
    b.add_argument("--registry", action="store_true", help="print the kernel support matrix (op, precision, target, kernel)")
    b.add_argument("--calibrate", action="store_true", help="measure HBM / GEMM / H2D floors")
    b.add_argument("--tp", type=int, default=1)
    b.add_argument("--record", action="store_true", help="append results to the bench store")
    b.add_argument("--suite", default=None,
                   help="run a measurement suite (spec, batch, sparse, tick, grpo, grpo-zero3; 'list' prints them); "
                        "flags the bench parser does not know go to the suite")
    b.add_argument("--record-line", default=None, metavar="FILE",
                   help="append the records of a bench.py JSON line (a file holding that line) to the bench store")

    g = sub.add_parser("generate", help="offline generation, one process per GPU")
    _add_model_flags(g)
    g.add_argument("--prompts", required=True)
    g.add_argument("--out", required=True)
    g.add_argument("--workers", type=int, default=1)
    g.add_argument("--max-tokens", "--max-new-tokens", dest="max_tokens", type=int, default=64)
    g.add_argument("--temperature", type=float, default=0.0)
    g.add_argument("--top-p", type=float, default=1.0)
    g.add_argument("--top-k", type=int, default=0)
    g.add_argument("--batch", type=int, default=8, help="prompts a worker keeps in flight")

    m = sub.add_parser("merge", help="merge fine-tuned checkpoints")
    m.add_argument("--base", required=True)
    m.add_argument("--tuned", nargs="+", default=None, help="fine-tuned checkpoint directories")
    m.add_argument("--specialists", type=lambda v: [x for x in v.split(",") if x], default=None,
                   help="the same as --tuned, comma-separated")
    m.add_argument("--out", required=True)
    m.add_argument("--method", default="average", choices=["average", "ties", "dare", "iso"])
    m.add_argument("--runs", default=None, help="run manifest directory (default: $TRL_RUNS or ./runs)")
    m.add_argument("--force", action="store_true", help="merge again even if a finished run with these inputs exists")
    m.add_argument("--json", action="store_true", help="print the run manifest as JSON")

    lg = sub.add_parser("ledger", help="list runs, show lineage, list devices")
    lg.add_argument("--runs", default=None, help="run manifest directory (default: $TRL_RUNS or ./runs)")
    lg.add_argument("--show", default=None)
    lg.add_argument("--devices", action="store_true")
    lg.add_argument("--time-to-score", type=float, default=None, metavar="SCORE",
                    help="per run: seconds of training until --metric first reached SCORE")
    lg.add_argument("--metric", default="eval_reward", help="logged metric that --time-to-score reads")
    return ap


def _device(args) -> str:
    if args.device:
        return args.device
    import torch
    return "cuda" if torch.cuda.is_available() else "cpu"


def ssd_slots(path: str, capacity_bytes: int, slot_bytes: int) -> int:
    """Pages the spill file may hold: ``capacity_bytes`` of them, or, with no capacity given, half of the
    free space of the file's filesystem; at least one, at most 2^24."""
    import shutil
    if capacity_bytes <= 0:
        capacity_bytes = shutil.disk_usage(os.path.dirname(os.path.abspath(path)) or ".").free // 2
    return int(max(1, min(1 << 24, capacity_bytes // max(1, slot_bytes))))


def _draft_window(args) -> int:
    w = args.draft_attn_window_tokens
    if w is None:
        w = int(os.environ.get("TRL_DRAFT_ATTN_WINDOW_TOKENS", "0") or 0)
    if w < 0:
        raise SystemExit("--draft-attn-window-tokens must not be negative")
    return int(w)


def cmd_serve(args) -> int:
    from . import memory
    from .config import get_config
    cfg = get_config(args.model)
    if args.dry_run:
        fp8 = args.kv_format == "fp8"
        host_pages = args.kv_cold_bytes // memory.kv_block_bytes(cfg, 1, fp8) if args.kv_cold_bytes else 0
        p = memory.plan(cfg, slots=args.slots, blocks=args.blocks, max_batched_tokens=args.max_batched_tokens,
                        planes=args.spec_width if (args.draft or args.draft_checkpoint) else 1, kv_fp8=fp8,
                        drafter=({"width": args.spec_width, **({"window": _draft_window(args)} if _draft_window(args) else {})}
                                 if args.draft == "block" else None),
                        indexer={} if (args.sparse_k and args.scorer == "learned") else None, host_pages=host_pages,
                        state_bytes=args.state_bytes, **({"device_bytes": args.device_free} if args.device_free else {}))
        print(json.dumps(memory.plan_json(p, args.device_free or memory.B200_BYTES)) if args.json else memory.memory_table(p))
        return 0
    from .engine import StepLimits
    from .factory import build_engine, build_model, make_ops
    from .server.app import create_app
    from .tokenizer import load_tokenizer
    dev = _device(args)
    if dev != "cpu" and not args.no_card_guard:
        try:
            from .parallel.health import card_guard
            card_guard(0)
        except ImportError:
            pass                      # no NVML binding in this environment: nothing to check with
    ops = make_ops(dev)
    model = build_model(cfg, dev, seed=args.seed, checkpoint=args.checkpoint, ops=ops if dev != "cpu" else None)
    drafter = None
    if args.draft_checkpoint:
        from .spec import load_drafter
        drafter = load_drafter(model, args.draft_checkpoint)
    elif args.draft:
        from .spec import BlockDrafter, ChainDrafter
        drafter = BlockDrafter(model) if args.draft == "block" else ChainDrafter(model)
    if drafter is not None and _draft_window(args) and hasattr(getattr(drafter, "cfg", None), "window"):
        drafter.cfg.window = _draft_window(args)     # a read window: rows kept and attended per request
    sparse = None
    if args.sparse_k:
        from .sparse import SparseConfig, SparseKV
        indexer = None
        if args.scorer == "learned":
            # the page indexer trained by `train --indexer-warmup --save-model DIR` replaces the Quest bound
            if not args.indexer:
                raise SystemExit("--scorer learned needs --indexer DIR (written by train --indexer-warmup --save-model)")
            from safetensors.torch import load_file
            from .sparse_index import LearnedIndexer
            indexer = LearnedIndexer(cfg, device=dev, n_q=model.dims.n_q)
            indexer.load_state_dict(load_file(os.path.join(args.indexer, "indexer.safetensors")))
        sparse = SparseKV(cfg, SparseConfig(args.sparse_k, max(1, args.sparse_window_tokens // 16),
                                            args.sparse_refresh_ticks, args.sparse_min_tokens), indexer=indexer)
    tok = load_tokenizer(args.tokenizer, cfg.vocab)
    eng = build_engine(model, ops, device=dev, blocks=args.blocks, slots=args.slots, max_ctx=args.max_ctx,
                       prefix=not args.no_prefix, graph=args.graph, spec_width=args.spec_width if drafter else 0,
                       drafter=drafter, sparse=sparse, kv_fp8=args.kv_format == "fp8",
                       reserve_bytes=args.device_reserve_mib << 20,
                       limits=StepLimits(args.max_batch, args.max_batched_tokens, max_inflight=args.max_inflight,
                                         long_prefill_cap=args.sparse_prefill_tokens,
                                         long_prefill_min=max(1, args.sparse_min_tokens)),
                       eos_id=tok.eos_id, detokenize=tok.decode, think_ids=getattr(tok, "think_ids", None))
    if args.state_bytes and hasattr(eng.prefix, "max_state_bytes"):
        eng.prefix.max_state_bytes = args.state_bytes          # device budget of resident GDN snapshots
    if args.kv_cold_bytes and hasattr(eng.prefix, "host"):
        from .kv_tiers import ColdSsdFile, DramSnapshots, HostKvPages
        ssd = None
        if args.cold_ssd_path:
            ssd = ColdSsdFile(args.cold_ssd_path, slot_bytes=eng.kv.block_bytes(),
                              slots=ssd_slots(args.cold_ssd_path, args.cold_ssd_bytes, eng.kv.block_bytes()))
        eng.prefix.host = HostKvPages(args.kv_cold_bytes, pin=dev != "cpu", cold=ssd)
        eng.prefix.dram = DramSnapshots(args.dram_bytes)
    if args.kv_store:
        from .kv_tiers import KvBootStore
        print(json.dumps({"kv_boot": KvBootStore(args.kv_store).boot(eng)}))
    if not args.no_warmup:
        eng.precapture((1,))
    if args.record_residency:
        from . import benchrec, memory
        res = memory.residency(eng)
        shape = {"model": cfg.name, "slots": args.slots, "tp": 1}
        for k, v in res.items():
            if v > 0:
                benchrec.append(benchrec.make_record(f"resident_{k}_bytes", v, shape, target="cpu" if dev == "cpu" else "b200"))
        print(json.dumps({"residency": res}), flush=True)
        if args.port == 0:            # record and leave: nothing is served
            return 0
    eng.run()
    app = create_app(eng, tok, cfg.name, pace=args.stream_pace, pace_depth=args.stream_pace_depth,
                     completion_timeout_s=args.completion_timeout_s)
    import uvicorn
    uvicorn.run(app, host=args.host, port=args.port, log_level="warning")
    return 0


def cmd_train(args) -> int:
    import torch
    from . import evals, rl
    from .checkpoint import load_adapter, save_adapter, save_checkpoint
    from .config import get_config
    from .factory import build_engine, build_model, make_ops
    from .ledger import Run, runs_dir
    from .optim import make_optimizer
    from .recipes import expand
    if getattr(args, "deterministic", False):
        os.environ.setdefault("CUBLAS_WORKSPACE_CONFIG", ":4096:8")
        torch.use_deterministic_algorithms(True, warn_only=True)
        torch.manual_seed(int(getattr(args, "seed", 0) or 0))
    over = {k: getattr(args, k) for k in ("steps", "group", "prompts_per_step", "max_tokens", "micro", "lora_rank",
                                          "lr", "optim", "reward")}
    if args.indexer_warmup:
        over["indexer_warmup"] = True
    if args.ctx:
        over["ctx"] = args.ctx
    if args.rl:
        over["rl"] = True
    if args.opd:
        over["opd"] = True
    flags = expand(args.recipe, over) if args.recipe else {**dict(model=args.model, steps=2, group=4, prompts_per_step=2,
                                                                  max_tokens=8, micro=0, lora_rank=0, lr=1e-5,
                                                                  optim="adamw", reward="even", rl=args.rl,
                                                                  opd=args.opd),
                                                           **{k: v for k, v in over.items() if v is not None}}
    curve_every = (args.eval_every or 0) if args.eval_gsm8k and not flags.get("lora_rank") else 0
    if curve_every and not args.dry_run:
        from .ledger import refuse_blind_curve
        refuse_blind_curve(args.eval_curve_n, args.curve_target_pt)
    if flags.get("allow_short_rollouts"):        # (a smoke recipe runs into its cap on purpose)
        args.allow_short_rollouts = True
    cfg = get_config(flags.get("model", args.model))
    if not args.dry_run and flags.get("reward") in ("gsm8k", "boxed") and not args.data and (flags.get("rl") or flags.get("opd")):
        raise SystemExit(f"reward {flags['reward']!r} scores completions against gold answers: give --data rows.jsonl "
                         "with {prompt, answer} rows")
    if args.dry_run:
        from . import memory
        rows = memory.train_plan(cfg, mode="lora" if flags.get("lora_rank") else "full", rank=flags.get("lora_rank") or 16,
                                 zero=args.zero, optimizer=flags.get("optim") or "adamw",
                                 micro_tokens=args.train_seq_len or (args.prompt_len + flags["max_tokens"]))
        width = max(len(k) for k in rows) + 1
        for k, v in rows.items():
            print(f"{k:{width}s} {v / memory.GIB:10.2f} GiB")
        print(f"{'total':{width}s} {sum(rows.values()) / memory.GIB:10.2f} GiB")
        return 0
    if flags.get("indexer_warmup"):
        # the warm-up runs the dense model on the reference backend and trains only the indexer
        from .factory import build_model as _bm
        from .sparse_index import LearnedIndexer, warmup
        model = _bm(cfg, "cpu", seed=args.seed, checkpoint=args.checkpoint)
        ix = LearnedIndexer(cfg, seed=args.seed, dim=args.indexer_di)
        if args.indexer_corpus:
            from .sparse_index import corpus_run, load_spans
            held = load_spans(args.indexer_corpus, "held", args.held_spans)
            control = load_spans(args.indexer_control_corpus, "held", args.held_spans) if args.indexer_control_corpus else None
            run = Run({"cmd": "train", **flags, "indexer_corpus": args.indexer_corpus, "k_pages": args.k_pages,
                       "q_samples": args.q_samples, "q_min_pos": args.q_min_pos, "di": args.indexer_di, "seed": args.seed,
                       "held_spans": args.held_spans, "control": args.indexer_control_corpus},
                      root=args.runs or runs_dir())
            out = corpus_run(model, ix, load_spans(args.indexer_corpus, "train"), held, args.k_pages, steps=flags["steps"],
                             lr=flags.get("lr") or 3e-3, q_samples=args.q_samples, q_min_pos=args.q_min_pos, seed=args.seed,
                             control=control, recall_threshold=args.recall_threshold)
            for i, kl in enumerate(out["kl_curve"]):
                run.log(step=i, kl=kl)
            run.log(**{f"recall_after_{k}": v for k, v in out["recall_after"].items()},
                    **{f"recall_before_{k}": v for k, v in out["recall_before"].items()})
            run.gate("worst_recall_after", out["worst_recall_after"], args.recall_threshold)
            print(json.dumps({k: v for k, v in out.items() if k != "kl_curve"} |
                             {"kl_first": out["kl_curve"][0], "kl_last": out["kl_curve"][-1]}))
            if args.save_model:
                from safetensors.torch import save_file
                os.makedirs(args.save_model, exist_ok=True)
                save_file(ix.state_dict(), os.path.join(args.save_model, "indexer.safetensors"))
                run.artifacts["indexer"] = args.save_model
            run.finish()
            return 0 if out["passed"] else 1
        g = torch.Generator().manual_seed(args.seed)
        seqs = [torch.randint(0, cfg.vocab, (flags.get("ctx") or 256,), generator=g) for _ in range(4)]
        run = Run({"cmd": "train", **flags}, root=args.runs or runs_dir())
        hist = warmup(model, ix, seqs, steps=flags["steps"], lr=flags.get("lr") or 3e-3)
        for i, kl in enumerate(hist):
            run.log(step=i, kl=kl)
        print(json.dumps({"kl_first": hist[0], "kl_last": hist[-1], "steps": len(hist)}))
        if args.save_model:
            from safetensors.torch import save_file
            os.makedirs(args.save_model, exist_ok=True)
            save_file(ix.state_dict(), os.path.join(args.save_model, "indexer.safetensors"))
            run.artifacts["indexer"] = args.save_model
        run.finish()
        return 0
    # everything that changes what the run computes is in its id: two runs that differ in one of these are
    # two runs, and the same command asked twice is handed the finished manifest
    inputs = {"cmd": "train", **flags, **({"data": args.data} if args.data else {}), "seed": args.seed,
              "checkpoint": args.checkpoint, "length_penalty": args.length_penalty, "judge": bool(args.judge),
              "max_think_tokens": args.max_think_tokens, "allow_short_rollouts": bool(args.allow_short_rollouts),
              "clip_eps": args.clip_eps, "kl_coef": args.kl_coef, "load_adapter": args.load_adapter,
              "prompt_len": args.prompt_len, "eval_gsm8k": args.eval_gsm8k, "eval_mmlu": args.eval_mmlu,
              "eval_n": args.eval_n, "eval_every": args.eval_every, "eval_curve_n": args.eval_curve_n,
              "eval_curve_seed": args.eval_curve_seed}
    if args.load_adapter and not args.lineage:
        # a run that starts from a saved adapter descends from the run that wrote it (looked up through the
        # manifests' artifacts, never guessed from the path)
        from .ledger import find_run_for_artifact
        args.lineage = find_run_for_artifact(args.load_adapter, args.runs or runs_dir())
    if not args.force:
        from .ledger import finished_run
        man = finished_run(inputs, args.lineage, args.runs or runs_dir())
        if man is not None:
            print(json.dumps(man if args.json else {"run": man["id"], "status": "done", "reused": True,
                                                    "hint": "--force trains it again"}, default=str), flush=True)
            return 0
    say = (lambda *a, **k: None) if args.json else print
    dev = _device(args)
    ops = make_ops(dev)
    model = build_model(cfg, dev, seed=args.seed, checkpoint=args.checkpoint, ops=ops if dev != "cpu" else None,
                        keep_master=not flags.get("lora_rank"))
    if flags.get("lora_rank"):
        model.add_lora(rank=flags["lora_rank"])
        if args.load_adapter:
            load_adapter(model, args.load_adapter)
    opt = make_optimizer(flags.get("optim", "adamw"), model.trainable(), flags["lr"])
    run = Run(inputs, root=args.runs or runs_dir(), parent=args.lineage)
    g = torch.Generator().manual_seed(args.seed)
    reward_fn = evals.REWARDS.get(flags["reward"], evals.reward_even)
    tok = eval_items = None
    if args.data or args.eval_gsm8k or args.eval_mmlu:
        from .tokenizer import load_tokenizer
        tok = load_tokenizer(args.tokenizer, cfg.vocab)

        def read_jsonl(path):
            with open(path) as f:
                rows = [json.loads(ln) for ln in f if ln.strip()]
            return [{"question": r.get("prompt", r.get("question")), "answer": str(r["answer"])} for r in rows]
    if args.data:
        items = read_jsonl(args.data)
        prompts = [tok.encode(it["question"]) for it in items]
        reward_fn = evals.make_text_reward(tok, {it["question"]: it["answer"] for it in items},
                                           kind="boxed" if flags.get("reward") == "boxed" else "gsm8k")
    else:
        prompts = [torch.randint(0, cfg.vocab, (args.prompt_len,), generator=g).tolist() for _ in range(64)]
    mmlu_items = curve_items = None
    if args.eval_gsm8k:
        every = read_jsonl(args.eval_gsm8k)
        eval_items = every[:args.eval_n]
        if curve_every:
            from .ledger import curve_rows
            curve_items = curve_rows(every, args.eval_curve_n, args.eval_curve_seed)
            if len(curve_items) < args.eval_curve_n:
                print(f"curve subset is {len(curve_items)} rows, not the {args.eval_curve_n} asked for", file=sys.stderr)
    if args.eval_mmlu:
        with open(args.eval_mmlu) as f:
            mmlu_items = [json.loads(ln) for ln in f if ln.strip()][:args.eval_n]
    eval_texts = [it["question"] for it in (eval_items or []) + (curve_items or [])] + \
                 [it["question"] + "\n" + "\n".join(it["choices"]) + "\nA. B. C. D. Answer:" for it in (mmlu_items or [])]
    longest = max(len(p) for p in prompts + [tok.encode(t) for t in eval_texts])
    eng = build_engine(model, ops, device=dev, slots=max(flags["group"] * flags["prompts_per_step"], 8) + 1,
                       max_ctx=max(args.prompt_len, longest) + max(flags["max_tokens"], args.eval_max_new_tokens if eval_texts else 0) + 32,
                       prefix=False, graph=False)

    def score(tag):
        if mmlu_items:
            eng.invalidate_weights()
            res = evals.evaluate(eng, tok, mmlu_items, kind="choice", max_tokens=min(8, args.eval_max_new_tokens))
            run.log(**{f"mmlu_{tag}_{k}": v for k, v in res.items()})
            say(json.dumps({f"mmlu_{tag}": res}), flush=True)
        if not eval_items:
            return None
        eng.invalidate_weights()
        res = evals.evaluate(eng, tok, eval_items, kind="gsm8k", max_tokens=args.eval_max_new_tokens)
        run.log(**{f"eval_{tag}_{k}": v for k, v in res.items()})
        say(json.dumps({f"eval_{tag}": res}), flush=True)
        return res

    def curve_point(step):
        from .ledger import binomial_se_pt
        eng.invalidate_weights()
        res = evals.evaluate(eng, tok, curve_items, kind="gsm8k", max_tokens=args.eval_max_new_tokens)
        pt = dict(curve_step=step, curve_accuracy=res["accuracy"], curve_n=res["n"],
                  curve_se_pt=round(binomial_se_pt(res["accuracy"], res["n"]), 2), curve_mean_tokens=res["mean_tokens"])
        run.log(**pt)
        say(json.dumps(pt), flush=True)

    def done():
        run.finish()
        if args.json:
            from .ledger import load_run
            print(json.dumps(load_run(run.id, run.root), default=str), flush=True)
        return 0
    judge = None
    if args.judge:
        from .tokenizer import load_tokenizer
        jtok = tok or load_tokenizer(args.tokenizer, cfg.vocab)

        def judge(prompt_ids, completions, rewards):
            cmp = evals.policy_compare(eng, jtok, question=jtok.decode(prompt_ids))
            return evals.judge_tiebreak(rewards, [jtok.decode(c) for c in completions], cmp)
    before = score("before")
    if flags.get("rl") and before:      # the base policy's own length against the rollout cap, both measured
        if before["mean_tokens"] < args.eval_max_new_tokens:      # (an eval that hit its own cap measured the cap)
            rl.refuse_short_rollouts(before["mean_tokens"], flags["max_tokens"], args.allow_short_rollouts)
    post = (lambda m: m.requantize_()) if not flags.get("lora_rank") else None
    if flags.get("lora_rank") and (flags.get("rl") or flags.get("opd")) and (args.eval_every or flags.get("eval_every")):
        # adapter run with evals, early stop and best-adapter save
        kw = dict(max_tokens=flags["max_tokens"], prompts_per_step=flags["prompts_per_step"])
        if not flags.get("opd"):
            kw.update(group=flags["group"], clip_eps=args.clip_eps, kl_coef=args.kl_coef, micro=flags.get("micro") or 0)
        out = rl.train_adapters(eng, model, prompts[:48], reward_fn, opt,
                                steps=flags["steps"], eval_prompts=prompts[48:], eval_every=args.eval_every or flags["eval_every"],
                                patience=flags.get("patience", args.patience), save_dir=args.save_model, run=run,
                                opd=bool(flags.get("opd")), **kw)
        say(json.dumps({k: v for k, v in out.items() if k != "history"}, default=str), flush=True)
        return done()
    if flags.get("opd"):
        loop = rl.opd_loop(eng, model, prompts, opt, steps=flags["steps"], max_tokens=flags["max_tokens"],
                           prompts_per_step=flags["prompts_per_step"])
    elif flags.get("rl"):
        loop = rl.grpo_loop(eng, model, prompts, reward_fn, opt,
                            steps=flags["steps"], group=flags["group"], prompts_per_step=flags["prompts_per_step"],
                            max_tokens=flags["max_tokens"], clip_eps=args.clip_eps, kl_coef=args.kl_coef,
                            micro=flags.get("micro") or 0, post_step=post, length_penalty=args.length_penalty, judge=judge,
                            max_think_tokens=args.max_think_tokens or None)
    else:
        data = iter(lambda: torch.randint(0, cfg.vocab, (2, args.prompt_len), generator=g), None)
        loop = iter(rl.pretrain(model, data, opt, steps=flags["steps"], lr=flags["lr"]))
    drift = rl.RolloutDrift(flags["max_tokens"]) if flags.get("rl") and not args.allow_short_rollouts else None
    if curve_items:
        curve_point(0)
    for m in loop:
        rows = m.pop("rollouts", None) if isinstance(m, dict) else None
        if rows:            # one JSON row per completion beside the manifest
            with open(os.path.join(run.dir, "rollouts.jsonl"), "a") as f:
                for r in rows:
                    f.write(json.dumps({"step": m["step"], **r}) + "\n")
        run.log(**{k: v for k, v in m.items() if not isinstance(v, (dict, list))})
        say(json.dumps(m, default=str), flush=True)
        if curve_items and (m["step"] + 1) % curve_every == 0:
            curve_point(m["step"] + 1)
        if drift is not None and "mean_completion_tokens" in m and not drift.update(m["mean_completion_tokens"], m["step"] + 1):
            run.gate("rollout_window_mean", drift.mean, drift.threshold, higher_is_better=False)
            print(drift.reason, file=sys.stderr, flush=True)
            break
    score("after")
    if args.save_model:
        if flags.get("lora_rank"):
            save_adapter(model, args.save_model)
        else:
            save_checkpoint(model, args.save_model)
        run.artifacts["model"] = args.save_model
    done()
    return 0 if run.status == "done" else 1


def cmd_bench(args) -> int:
    from . import kernel_cost as kc
    from .calibration import calibrate, load_peaks
    from .config import get_config
    if args.suite:
        from . import suites
        if args.suite == "list":
            print("\n".join(sorted(suites.SUITES)))
            return 0
        return suites.run(args.suite, getattr(args, "suite_args", []))
    if args.record_line:
        from . import benchrec
        with open(args.record_line) as f:
            lines = [ln for ln in f.read().splitlines() if ln.startswith("{")]
        n = 0
        from .calibration import load_peaks
        for rec in benchrec.records_from_bench_line(json.loads(lines[-1]), hbm_gbs=load_peaks().hbm_gbs):
            benchrec.append(rec)
            n += 1
        print(f"appended {n} records to {benchrec.store_path()}")
        return 0
    cfg = get_config(args.model)
    if args.calibrate:
        import dataclasses
        pk = calibrate(_device(args))
        print(json.dumps(dataclasses.asdict(pk)))
        if args.record:             # the floors join the bench store, where `ledger --devices` reads them
            from . import benchrec
            benchrec.append(benchrec.make_record("hbm_copy_gbs", pk.hbm_gbs, {}))
            benchrec.append(benchrec.make_record("bf16_gemm_tflops", pk.bf16_tflops, {}))
        return 0
    if args.registry:
        from .ops import registry as R
        print(f"{'op':28s} {'precision':9s} {'target':6s} {'kernel':60s} source")
        for (precision, arch), table in sorted(R._CELLS.items()):
            for op, k in sorted(table.items()):
                print(f"{op:28s} {precision:9s} {arch:6s} {k.name[:60]:60s} {k.source}")
        return 0
    pk = load_peaks()
    if args.kernels:
        from .calibration import peaks_for
        try:
            pk = peaks_for(args.device_name)
        except KeyError as e:
            raise SystemExit(str(e.args[0]))
        print(f"# floors ({pk.source}): {pk.hbm_gbs:.0f} GB/s memory, {pk.bf16_tflops:.0f} TFLOP/s bf16, {pk.nvlink_gbs:.0f} GB/s link")
        if args.prefill:
            print(kc.table(kc.prefill_rows(cfg, args.prefill, args.tp), pk.hbm_gbs, 4 * pk.bf16_tflops, pk.nvlink_gbs))
            return 0
        rows = kc.tick_rows(cfg, kc.TickShape(batch=int(args.batches.split(",")[0]), ctx=args.context or args.prompt_len,
                                              tp=args.tp))
        print(kc.table(rows, pk.hbm_gbs, pk.bf16_tflops, pk.nvlink_gbs))
        print(kc.table(kc.prefill_rows(cfg, args.prompt_len, args.tp), pk.hbm_gbs, 4 * pk.bf16_tflops, pk.nvlink_gbs))
        return 0
    import time
    import torch
    from .engine import SamplingParams
    from .factory import build_engine, build_model, make_ops
    dev = _device(args)
    ops = make_ops(dev)
    model = build_model(cfg, dev, seed=args.seed, checkpoint=args.checkpoint, ops=ops if dev != "cpu" else None)
    out = []
    for b in [int(x) for x in args.batches.split(",")]:
        eng = build_engine(model, ops, device=dev, slots=b + 1, max_ctx=args.prompt_len + args.gen + 32, prefix=False)
        g = torch.Generator().manual_seed(1)
        prompts = [torch.randint(0, cfg.vocab, (args.prompt_len,), generator=g).tolist() for _ in range(b)]
        for _ in range(3):
            eng.generate(prompts, SamplingParams(max_tokens=min(4, args.gen), ignore_eos=True))
        t0 = time.perf_counter()
        res = eng.generate(prompts, SamplingParams(max_tokens=args.gen, ignore_eos=True))
        dt = time.perf_counter() - t0
        ttft = sum(r.ttft_s for r in res) / b
        rec = {"batch": b, "prefill_tok_s": round(b * args.prompt_len / max(ttft, 1e-9), 1),
               "decode_tok_s": round(b * (args.gen - 1) / max(dt - ttft, 1e-9), 1)}
        out.append(rec)
        if args.record:
            from . import benchrec
            benchrec.append(benchrec.make_record("decode_tok_s", rec["decode_tok_s"],
                                                 dict(model=cfg.name, batch=b, ctx=args.prompt_len, tp=args.tp)))
    print(json.dumps(out))
    return 0


def cmd_generate(args) -> int:
    from .generate import generate
    files = generate(args.model, args.prompts, args.out, workers=args.workers, device=_device(args),
                     max_tokens=args.max_tokens, temperature=args.temperature, checkpoint=args.checkpoint,
                     tokenizer_path=args.tokenizer, seed=args.seed, top_p=args.top_p, top_k=args.top_k, batch=args.batch)
    print(json.dumps({"files": files}))
    return 0


def cmd_merge(args) -> int:
    from .ledger import Run, find_run_for_artifact, finished_run, load_run, runs_dir
    from .merge import merge_checkpoints
    tuned = list(args.tuned or []) + list(args.specialists or [])
    if not tuned:
        raise SystemExit("merge needs --tuned DIR [DIR ...] or --specialists DIR,DIR")
    root = args.runs or runs_dir()
    inputs = {"cmd": "merge", "base": args.base, "specialists": tuned, "method": args.method, "out": args.out}
    prev = None if args.force else finished_run(inputs, None, root)
    if prev is not None and os.path.isdir(args.out):
        print(json.dumps(prev, default=str) if args.json else
              json.dumps({"run": prev["id"], "status": "done", "reused": True, "hint": "--force merges again"}))
        return 0
    # lineage goes through the runs that wrote the inputs; a directory no run lists contributes no parent
    parents = [pid for pid in (find_run_for_artifact(p, root) for p in [args.base] + tuned) if pid is not None]
    run = Run(inputs, root=root, parents=parents)
    n = merge_checkpoints(args.base, tuned, args.out, args.method)
    run.log(tensors=n)
    run.artifacts["model"] = args.out
    run.finish()
    print(json.dumps(load_run(run.id, root), default=str) if args.json else
          json.dumps({"tensors": n, "out": args.out, "run": run.id, "parents": parents}))
    return 0


def cmd_ledger(args) -> int:
    from . import ledger
    if args.devices:
        from . import benchrec
        print(json.dumps(ledger.devices(), indent=1))
        print(ledger.format_device_sections(ledger.device_sections(benchrec.load(benchrec.store_path()))))
        return 0
    if args.show:
        print(json.dumps({"run": ledger.load_run(args.show, args.runs), "lineage": ledger.lineage(args.show, args.runs)},
                         indent=1))
        return 0
    for r in ledger.list_runs(args.runs):
        line = f"{r['id']}  {r['status']:12s} {r['seconds']:8.1f}s  {r['inputs'].get('recipe') or r['inputs'].get('cmd', '')}"
        if args.time_to_score is not None:
            t = ledger.time_to_score(r, args.metric, args.time_to_score)
            line += f"  {args.metric}>={args.time_to_score:g}: " + (f"{t:.1f}s" if t is not None else "never")
        print(line)
    return 0


def main(argv: Optional[List[str]] = None) -> int:
    args, rest = build_parser().parse_known_args(argv)
    if rest and not (args.cmd == "bench" and args.suite):
        build_parser().parse_args(argv)          # unknown flags are an error everywhere else
    args.suite_args = rest
    return {"serve": cmd_serve, "train": cmd_train, "bench": cmd_bench, "generate": cmd_generate,
            "merge": cmd_merge, "ledger": cmd_ledger}[args.cmd](args)


if __name__ == "__main__":
    sys.exit(main())
