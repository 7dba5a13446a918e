"""Timeline of one decode tick: where the time between two dependent kernels goes.

    python -m tilerl_b200.build --trace
    TRL_TRACE_LIB=1 python -m tilerl_b200.utils.tick_trace [--model qwen38-27b] [--ctx 512]
    TRL_TRACE_LIB=1 python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 \
        -m tilerl_b200.utils.tick_trace          # tensor-parallel tick, rank 0's timeline

The ``-DTRL_TRACE`` build records, per launch, when CTA 0 entered the kernel and when its
dependency wait ended.  The wait of launch ``i + 1`` ends when launch ``i`` has completed, so
``dep[i + 1] - dep[i]`` is launch ``i``'s share of the tick's critical path; ``dep[i] -
entry[i]`` says how early the launch was resident (overlap won by programmatic dependent launch).
The tool replays the captured B = 1 decode graph, reads the records and prints the per-kernel sums.
"""
from __future__ import annotations

import argparse
import collections
import json

import numpy as np
import torch

KINDS = {2: "gdn_scan", 3: "attn_prep", 4: "attn_split", 5: "attn_combine", 6: "gemv_bf16(lm_head)", 7: "embedding",
         10: "allreduce_finish", 12: "gdn_prep", 100: "gemv2 store", 101: "gemv2 store+coop", 102: "gemv2 residual",
         104: "gemv2 swiglu", 105: "gemv2 swiglu+coop", 106: "gemv2 store_f32", 108: "gemv2 push", 109: "gemv2 push+coop", 120: "gemv2 chain", 0: "other"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="qwen38-27b")
    ap.add_argument("--ctx", type=int, default=512)
    ap.add_argument("--ticks", type=int, default=4)
    args = ap.parse_args()
    from tilerl_b200.config import get_config
    from tilerl_b200.factory import build_engine, build_model, make_ops
    from tilerl_b200.engine import SamplingParams
    from tilerl_b200.ops import native
    import os
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", 0)))
    torch.cuda.set_device(dev)
    cfg = get_config(args.model)
    comm = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
        from tilerl_b200.parallel.symm import SymmComm
        comm = SymmComm.create(dist.group.WORLD, dev)
    ops = make_ops(dev, tp_comm=comm)
    model = build_model(cfg, dev, seed=0, tp_rank=rank, tp=world, ops=ops)
    eng = build_engine(model, ops, slots=2, max_ctx=args.ctx + 64, graph=True, prefix=False)
    g = torch.Generator().manual_seed(1)
    prompt = torch.randint(0, cfg.vocab, (args.ctx,), generator=g).tolist()
    eng.generate([prompt], SamplingParams(max_tokens=4, ignore_eos=True))      # captures the graph
    torch.cuda.synchronize()
    buf = np.zeros((8192, 16), dtype=np.uint64)
    native.lib().trl_trace_read(buf.ctypes.data, 8192, 1)                       # reset
    eng.generate([prompt], SamplingParams(max_tokens=args.ticks + 1, ignore_eos=True))
    torch.cuda.synchronize()
    n = native.lib().trl_trace_read(buf.ctypes.data, 8192, 1)
    if n <= 0:
        raise SystemExit("no records: load the -DTRL_TRACE build with TRL_TRACE_LIB=1")
    rec = buf[:n].astype(np.int64)
    # the last tick: from the last embedding launch on
    emb = [i for i in range(n) if rec[i, 0] == 7]
    if len(emb) < 2:
        raise SystemExit("fewer than two ticks recorded")
    a, b = emb[-2], emb[-1]
    tick = rec[a:b + 1]
    dep = tick[:, 2]
    share = collections.OrderedDict()
    early = collections.OrderedDict()
    phases = collections.OrderedDict()
    for i in range(len(tick) - 1):
        name = KINDS.get(int(tick[i, 0]), f"kind {int(tick[i, 0])}")
        d = share.setdefault(name, [0, 0.0])
        d[0] += 1
        d[1] += (dep[i + 1] - dep[i]) / 1e3
        e = early.setdefault(name, 0.0)
        early[name] = e + (dep[i] - tick[i, 1]) / 1e3
        # phases of CTA 0 after its wait (kernels that mark them), and what follows its exit
        if tick[i, 4] and tick[i, 5] and tick[i, 3]:
            ph = phases.setdefault(name, [0, 0.0, 0.0, 0.0, 0.0, 0.0])
            ph[0] += 1
            ph[1] += (tick[i, 4] - dep[i]) / 1e3          # dependency resolved -> activation staged
            ph[2] += (tick[i, 5] - tick[i, 4]) / 1e3      # main loop of CTA 0's first warp
            ph[3] += (tick[i, 3] - tick[i, 5]) / 1e3      # epilogue of CTA 0
            if tick[i + 1, 6]:
                ph[4] += (int(tick[i + 1, 6]) - int(tick[i, 3])) / 1e3    # last CTA's exit after CTA 0's
                ph[5] += (int(dep[i + 1]) - int(tick[i + 1, 6])) / 1e3    # last exit -> next launch released
    # chained launches (kind 120): marks 0..9 = per op (past its barrier, row staged, main loop done)
    chain = [tick[i] for i in range(len(tick) - 1) if int(tick[i, 0]) == 120 and tick[i, 4]]
    if chain:
        c = np.array(chain, dtype=np.float64)
        marks = np.concatenate([c[:, 4:6], c[:, 8:16]], axis=1)            # marks 0..9
        rel = (marks - c[:, 2:3]) / 1e3
        rel[marks == 0] = np.nan
        names = [f"op{j}:{w}" for j in range(4) for w in ("past_barrier", "staged", "main_done")][:10]
        out_chain = {nm: round(float(np.nanmean(rel[:, k])), 2) for k, nm in enumerate(names) if not np.all(np.isnan(rel[:, k]))}
        out_chain["exit"] = round(float(np.mean((c[:, 3] - c[:, 2]) / 1e3)), 2)
    else:
        out_chain = None
    total = (dep[-1] - dep[0]) / 1e3
    out = {"tick_us": round(total, 1), "launches": len(tick) - 1,
           "critical_path_us": {k: {"n": v[0], "sum": round(v[1], 1), "avg": round(v[1] / v[0], 2),
                                    "resident_before_dep_avg": round(early[k] / v[0], 2)}
                                for k, v in sorted(share.items(), key=lambda kv: -kv[1][1])}}
    out["phases_us_avg"] = {k: dict(zip(("staged", "main_loop", "epilogue", "last_cta_after_cta0", "release_after_last_exit"),
                                        [round(x / v[0], 2) for x in v[1:]])) for k, v in phases.items()}
    if out_chain:
        out["chain_marks_us_after_dependency_avg"] = out_chain
    if rank == 0:
        print(json.dumps(out))
        print("tick_trace done")
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
