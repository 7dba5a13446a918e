"""GRPO step with a ZeRO-3 trainer and a tensor-parallel NVFP4 rollout engine on the same
ranks (one process per GPU, launched by torchrun):

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        -m tilerl_b200.suites.grpo_zero3 --model qwen38-27b --prompts 8 --group 8 \
        --prompt-len 256 --gen 512 --steps 2

Every rank holds (a) its TP shard of the NVFP4 rollout weights and (b) its ZeRO-3 shard of the
fp32 master weights and Adam moments.  A step is: rollout of prompts x group sequences through
the TP engine (all ranks run the same ticks), each rank trains on its own slice of the
sequences (gradients reduce-scattered by the peer-memory kernels), AdamW on the shards, and the
in-place resync of the rollout weights.  Times are device-synchronised and reported as the max
over ranks.  Synthetic token prompts, random-init weights, reward = (sum of last 4 ids) % 7 == 0.
"""
from __future__ import annotations

import argparse
import json
import os
import time

import torch
import torch.distributed as dist


def main(argv=None):
    ap = argparse.ArgumentParser(prog="tilerl_b200.suites.grpo_zero3")
    ap.add_argument("--model", default="qwen38-27b")
    ap.add_argument("--prompts", type=int, default=8)
    ap.add_argument("--group", type=int, default=8)
    ap.add_argument("--prompt-len", type=int, default=256)
    ap.add_argument("--gen", type=int, default=512)
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--lr", type=float, default=1e-6)
    ap.add_argument("--comm", default="p2p", choices=["p2p", "nccl"])
    ap.add_argument("--micro", type=int, default=0, help="sequences per micro-batch on a rank (0: all)")
    args = ap.parse_args(argv)
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    group = dist.group.WORLD if world > 1 else None
    from tilerl_b200 import evals, rl
    from tilerl_b200.config import get_config
    from tilerl_b200.engine import SamplingParams
    from tilerl_b200.factory import build_engine, build_model, make_ops
    from tilerl_b200.parallel.resync import resync
    from tilerl_b200.parallel.zero3 import P2PComm, Zero3
    cfg = get_config(args.model)
    comm = None
    if world > 1:
        from tilerl_b200.parallel.symm import SymmComm
        comm = SymmComm.create(group, dev, hmax=cfg.hidden, tmax=max(512, args.prompt_len))
    ops = make_ops(dev, tp_comm=comm)
    ops.gemv_tokens = 4
    t0 = time.perf_counter()
    rollout = build_model(cfg, dev, seed=0, tp_rank=rank, tp=world, ops=ops)
    trainer = build_model(cfg, dev, seed=0, master_only=True)       # full masters, sharded next
    numel = sum(p.numel() for p in trainer.trainable("full").values())
    per_unit = max(sum(p.numel() for n, p in trainer.trainable("full").items() if n.startswith(f"master.L{i}.")
                       or n.startswith(f"L{i}.")) for i in range(cfg.n_layers))
    zcomm = P2PComm(group, dev, cap_bytes=per_unit * 2 + (1 << 20)) if (world > 1 and args.comm == "p2p") else None
    z = Zero3(trainer, group, lr=args.lr, max_norm=1.0, comm=zcomm)
    torch.cuda.empty_cache()
    build_s = time.perf_counter() - t0
    n_seq = args.prompts * args.group
    eng = build_engine(rollout, ops, device=dev, slots=n_seq + 1, max_ctx=args.prompt_len + args.gen + 64,
                       prefix=False, graph=True)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, cfg.vocab, (args.prompt_len,), generator=g).tolist() for _ in range(args.prompts)]
    rows = []
    for step in range(args.steps):
        torch.cuda.synchronize()
        t_a = time.perf_counter()
        rids = []
        for pi, p in enumerate(prompts):
            for gi in range(args.group):
                rids.append(eng.submit(p, SamplingParams(max_tokens=args.gen, temperature=1.0, logprobs=True,
                                                         seed=(step * 1009 + pi) * 131 + gi)))
        results = rl.drain(eng, rids)
        torch.cuda.synchronize()
        t_b = time.perf_counter()
        comps = [r.tokens if r is not None else [] for r in results]
        rewards = [float(evals.reward_mod7(prompts[i // args.group], c)) for i, c in enumerate(comps)]
        adv = rl.group_advantages(rewards, args.group, [len(c) > 0 for c in comps])
        mine = list(range(rank, n_seq, world))                       # this rank's slice of the sequences
        seqs = [list(prompts[i // args.group]) + comps[i] for i in mine]
        plens = [len(prompts[i // args.group]) for i in mine]
        slens = [len(s) for s in seqs]
        ids = rl.pad_batch(seqs).to(dev)
        stats = rl.policy_step(trainer, ids, plens, slens, adv[mine], z, clip_eps=0.2, kl_coef=0.0, max_norm=0.0,
                               micro=args.micro, checkpoint_layers=True, on_grad=z.on_grad, hook=z, fused_ce=True)
        torch.cuda.synchronize()
        t_c = time.perf_counter()
        rs = resync(z, rollout, quantize=ops.quantize_new, refresh=ops.refresh_weight, engine=eng)
        torch.cuda.synchronize()
        t_d = time.perf_counter()
        t = torch.tensor([t_b - t_a, t_c - t_b, t_d - t_c, t_d - t_a], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        row = dict(step=step, rollout_s=float(t[0]), train_s=float(t[1]), resync_s=float(t[2]), total_s=float(t[3]),
                   reward=sum(rewards) / len(rewards), loss=stats["loss"], completion_tokens=sum(len(c) for c in comps),
                   resync_bytes=rs["bytes"])
        rows.append(row)
        if rank == 0:
            print(json.dumps(row), flush=True)
    if rank == 0:
        last = rows[-1]
        print(json.dumps(dict(metric="grpo_step_s", value=round(last["total_s"], 3), n_gpus=world, model=cfg.name,
                              rollout_s=round(last["rollout_s"], 3), train_s=round(last["train_s"], 3),
                              resync_s=round(last["resync_s"], 3), prompts=args.prompts, group=args.group,
                              gen=args.gen, trainable_params=numel, zero_comm=args.comm if world > 1 else "none",
                              zero_stats=z.stats, build_s=round(build_s, 1),
                              peak_gib=round(torch.cuda.max_memory_allocated() / 2 ** 30, 2))))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
