"""Time GRPO steps on one GPU: rollout through the engine, policy update on the tape.

    python -m tilerl_b200.suites.grpo --model qwen38-27b --group 8 --prompts 1 \
        --prompt-len 256 --gen 1024 --lora 16 --micro 1 --steps 2

Prints one JSON line per step with the phase timings (rollout / score / train / invalidate) and
a final summary line.  Prompts are uniform-random token ids, weights random-init, the reward is
the deterministic ``sum(last 4 ids) % 7 == 0`` of the synthetic configs.
"""
from __future__ import annotations

import argparse
import json
import time

import torch


def main(argv=None):
    ap = argparse.ArgumentParser(prog="tilerl_b200.suites.grpo")
    ap.add_argument("--model", default="qwen38-27b")
    ap.add_argument("--group", type=int, default=8)
    ap.add_argument("--prompts", type=int, default=1)
    ap.add_argument("--prompt-len", type=int, default=256)
    ap.add_argument("--gen", type=int, default=1024)
    ap.add_argument("--lora", type=int, default=16)
    ap.add_argument("--micro", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--lr", type=float, default=1e-6)
    ap.add_argument("--graph", type=int, default=1)
    args = ap.parse_args(argv)
    from tilerl_b200 import evals, rl
    from tilerl_b200.config import get_config
    from tilerl_b200.factory import build_engine, build_model, make_ops
    from tilerl_b200.optim import AdamW
    dev = torch.device("cuda", 0)
    cfg = get_config(args.model)
    ops = make_ops(dev)
    ops.gemv_tokens = 4          # batched rollout: 5..8 rows take the tensor-core GEMM
    t0 = time.perf_counter()
    model = build_model(cfg, dev, seed=0, ops=ops, keep_master=args.lora == 0)
    if args.lora:
        model.add_lora(rank=args.lora)
    build_s = time.perf_counter() - t0
    n_seq = args.group * args.prompts
    eng = build_engine(model, ops, device=dev, slots=n_seq + 1, max_ctx=args.prompt_len + args.gen + 64,
                       prefix=False, graph=bool(args.graph))
    opt = AdamW(model.trainable(), lr=args.lr)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, cfg.vocab, (args.prompt_len,), generator=g).tolist() for _ in range(16)]
    post = (lambda m: m.requantize_()) if not args.lora else None
    rows = []
    for m in rl.grpo_loop(eng, model, prompts, evals.reward_mod7, opt, steps=args.steps, group=args.group,
                          prompts_per_step=args.prompts, max_tokens=args.gen, clip_eps=0.2, kl_coef=0.0,
                          micro=args.micro, post_step=post, checkpoint_layers=True, fused_ce=True):
        torch.cuda.synchronize()
        rows.append(m)
        print(json.dumps({k: v for k, v in m.items() if k != "rollouts"}, default=float), flush=True)
    last = rows[-1]["timings"]
    print(json.dumps(dict(metric="grpo_step_s", value=round(last["total"], 3), rollout_s=round(last["rollout"], 3),
                          train_s=round(last["train"], 3), completion_tokens=rows[-1]["completion_tokens"],
                          model=cfg.name, group=args.group, prompts=args.prompts, gen=args.gen, lora=args.lora,
                          micro=args.micro, build_s=round(build_s, 1),
                          peak_gib=round(torch.cuda.max_memory_allocated() / 2 ** 30, 2))))


if __name__ == "__main__":
    main()
