"""Headline benchmark: B=1 greedy decode tok/s (and prefill tok/s) of the 27B hybrid
model in NVFP4, 512-token prompt / 64 output tokens, at TP = number of GPUs.

One *step* is one request.  Two measurements per run:

* ``value`` (device-timed): CUDA events around the prefill forward and around the
  63 captured decode ticks replayed back to back with the device-side advance
  kernel (no host in the loop); max over ranks.
* ``e2e``: the same requests through the public engine API
  (``Engine.submit`` / ``step`` / ``take``): every tick copies its inputs from
  pinned host memory and reads the sampled token back.

Weights are random-init N(0, 0.02) quantised to NVFP4; prompts are uniform-random
token ids.  Each decode tick streams ~16 GB of weights, far above the 126 MB L2,
so no explicit L2 flush is needed between iterations.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
import zlib

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

BASELINE_DECODE_TOK_S = 92.4     # reference README.md:12, 1x H20
BASELINE_PREFILL_TOK_S = 2689.8  # reference README.md:12, 1x H20
PROMPT_LEN, GEN_LEN = 512, 64


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "200",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:  # noqa: BLE001
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=3)
        except Exception:  # noqa: BLE001
            self.proc.kill()
        sm, mx, reasons, power = [], [], set(), []
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            p = [x.strip() for x in ln.split(",")]
            if len(p) < 9:
                continue
            try:
                sm.append(float(p[1])), mx.append(float(p[2])), power.append(float(p[3]))
            except ValueError:
                continue
            for name, v in zip(names, p[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(power) if power else None, "samples": len(sm), "reasons": sorted(reasons)}


REF_DIR = os.path.join(ROOT, "baseline", "_ref")

_REF_CHILD = r"""
import json, os, sys, time, traceback
sys.path.insert(0, sys.argv[1])
prompt_len, gen, steps, warmup = (int(v) for v in sys.argv[2:6])
stage = "import"
try:
    import torch
    import tilerl, tilerl_kernels                      # the unmodified reference packages
    from tilerl_kernels.backend import get_backend
    from tilerl import engine as engine_mod
    from tilerl import model as model_mod
    from tilerl import config as config_mod
    from tilerl.build import build_model, build_serving_engine
    if not torch.cuda.is_available():
        raise RuntimeError("no CUDA device in this process")
    stage = "get_backend"
    backend = get_backend()
    # the stock serving path on the reference's own smallest model first: it compiles the kernel
    # cell of this device; only if that works is the 27B worth building (108 GB of fp32 on the host)
    stage = "stock serving path on its tiny model (build_model, build_serving_engine, submit, step)"
    cfg, model = build_model("tiny", seed=0)
    engine = build_serving_engine(cfg, model, backend)
    g = torch.Generator().manual_seed(0)
    rid = engine.submit(torch.randint(0, cfg.vocab_size, (16,), generator=g).tolist(),
                        engine_mod.SamplingParams(temperature=0.0, top_p=1.0, max_new_tokens=2, seed=0))
    for _ in range(8):
        engine.step()
        if rid in engine.poll():
            break
    stage = "27B random-init build (model.build_random(qwen38_27b()))"
    cfg = config_mod.qwen38_27b()
    model = model_mod.build_random(cfg, seed=0, fuse_projections=True)
    engine = build_serving_engine(cfg, model, backend)
    stage = "27B timed requests"
    def request(n_new):
        rid = engine.submit(torch.randint(0, cfg.vocab_size, (prompt_len,), generator=g).tolist(),
                            engine_mod.SamplingParams(temperature=0.0, top_p=1.0, max_new_tokens=n_new, seed=0))
        torch.cuda.synchronize(); t0 = time.perf_counter()
        engine.step()
        torch.cuda.synchronize(); t1 = time.perf_counter()
        n = 0
        while rid not in engine.poll():
            engine.step(); n += 1
        torch.cuda.synchronize(); t2 = time.perf_counter()
        return t1 - t0, t2 - t1, n
    for _ in range(max(3, warmup)):
        request(2)
    pre = dec = 0.0; ticks = 0
    for _ in range(steps):
        a, b, n = request(gen)
        pre += a; dec += b; ticks += n
    print(json.dumps({"ok": True, "decode_tok_s": ticks / dec, "prefill_tok_s": steps * prompt_len / pre,
                      "ms_per_step": (pre + dec) / steps * 1e3, "target": str(getattr(backend, "target", "?"))}))
except BaseException as e:                              # SystemExit included: the stock path exits on errors
    tail = traceback.format_exc().strip().splitlines()[-1]
    print(json.dumps({"ok": False, "stage": stage, "error": f"{type(e).__name__}: {str(e)[:300]}", "tail": tail[:300]}))
"""


def reference_arm(args):
    """Run the UNMODIFIED reference (a plain copy of its two pure-Python packages under
    ``baseline/_ref``; its ``pip install`` needs the ``uv_build`` backend, which the image lacks)
    through its own public API and stock serving path -- ``get_backend``, ``build_model`` /
    ``model.build_random``, ``build_serving_engine``, ``submit`` / ``step`` / ``poll``, the calls
    its ``tilerl bench`` makes (``src/tilerl/bench.py:246-299``) -- in a child process, and report
    either its numbers or the exception it raised."""
    out = {"impl": "reference"}
    if not os.path.isdir(os.path.join(REF_DIR, "tilerl")) or not os.path.isdir(os.path.join(REF_DIR, "tilerl_kernels")):
        out["unavailable"] = "baseline/_ref holds no copy of the reference packages (tilerl, tilerl_kernels)"
        print(json.dumps(out))
        return
    if args.gpus > 1:
        out["unavailable"] = ("the reference serves on one card per process (src/tilerl/tensor_parallel.py:20-24: "
                              "TP is a training path run eagerly); its single-card arm is the N=1 run")
        print(json.dumps(out))
        return
    env = {**os.environ, "PYTHONPATH": REF_DIR, "TILERL_TARGET": os.environ.get("TILERL_TARGET", "cuda")}
    try:
        r = subprocess.run([sys.executable, "-c", _REF_CHILD, REF_DIR, str(args.prompt_len), str(args.gen),
                            str(args.steps), str(args.warmup)], capture_output=True, text=True, timeout=1500, env=env)
        line = [ln for ln in r.stdout.strip().splitlines() if ln.startswith("{")]
        res = json.loads(line[-1]) if line else {"ok": False, "stage": "child process",
                                                  "error": (r.stderr.strip().splitlines() or ["no output"])[-1][:300]}
    except subprocess.TimeoutExpired:
        res = {"ok": False, "stage": "child process", "error": "no result within 1500 s"}
    if res.get("ok"):
        out.update({"metric": "decode_tok_s_b1_27b_nvfp4_prompt512_gen64", "value": round(res["decode_tok_s"], 2),
                    "unit": "tok/s", "n_gpus": 1, "steps": args.steps, "warmup": max(3, args.warmup),
                    "ms_per_step": round(res["ms_per_step"], 3), "higher_is_better": True,
                    "prefill_tok_s": round(res["prefill_tok_s"], 1), "target": res.get("target")})
    else:
        out["unavailable"] = (f"reference's stock path failed at [{res.get('stage')}]: {res.get('error')}"
                              + (f" | {res['tail']}" if res.get("tail") and res["tail"] not in res.get("error", "") else ""))
    print(json.dumps(out))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--model", default="qwen38-27b")
    ap.add_argument("--prompt-len", type=int, default=PROMPT_LEN)
    ap.add_argument("--gen", type=int, default=GEN_LEN)
    ap.add_argument("--no-control", action="store_true", help="skip the unfused same-box control at N > 1")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm(args)
    if args.impl not in ("ours", "unfused"):
        raise SystemExit("--impl is one of: ours, unfused, reference")

    import torch
    import torch.distributed as dist
    from tilerl_b200.batch import Batch
    from tilerl_b200.config import get_config
    from tilerl_b200.engine import SamplingParams
    from tilerl_b200.factory import build_engine, build_model, make_ops
    from tilerl_b200.ops import native

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    comm = None
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
        from tilerl_b200.parallel.symm import NcclComm, SymmComm
        comm = NcclComm(dist.group.WORLD, dev) if args.impl == "unfused" else SymmComm.create(dist.group.WORLD, dev)
    W = max(3, args.warmup)
    K = args.steps
    cfg = get_config(args.model)
    ops = make_ops(dev, tp_comm=comm)
    t0 = time.time()
    model = build_model(cfg, dev, seed=0, tp_rank=rank, tp=world, ops=ops)
    torch.cuda.synchronize()
    build_s = time.time() - t0
    max_ctx = 1024
    unfused = args.impl == "unfused" and world > 1
    eng = build_engine(model, ops, slots=2, max_ctx=max_ctx, graph=not unfused, prefix=False)
    runner = eng.graph
    g = torch.Generator().manual_seed(1234)
    prompts = [torch.randint(0, cfg.vocab, (args.prompt_len,), generator=g, dtype=torch.int32).pin_memory()
               for _ in range(W + K)]
    sp = SamplingParams(max_tokens=args.gen, ignore_eos=True)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-timed arm ---------------------------------------------------------------
    nblk = (args.prompt_len + args.gen + 16) // 16
    blocks = [eng.kv.alloc_block() for _ in range(nblk)]
    slot = eng.states.alloc_slot()
    ticks = args.gen - 1
    ev = lambda: torch.cuda.Event(enable_timing=True)

    def device_request(prompt_cpu):
        eng.states.states[slot].zero_()
        eng.states.ring[slot].zero_()
        eng.states.cur[slot] = 0
        toks = prompt_cpu.tolist()
        e0, e1, e2, e3 = ev(), ev(), ev(), ev()
        batch = Batch.build([dict(tokens=toks, start=0, blocks=blocks, slot=slot)], dev)
        e0.record()
        logits = model.forward(batch, ops, eng.kv, eng.states)
        tok = ops.argmax(logits)
        e1.record()
        first = int(tok[0])
        if unfused:
            # library collectives are not part of a captured tick here: eager ticks, the token read back
            # each time (what the reference's tensor-parallel ticks do)
            e2.record()
            for i in range(ticks):
                b1 = Batch.build([dict(tokens=[first], start=args.prompt_len + i, blocks=blocks, slot=slot)], dev)
                first = int(ops.argmax(model.forward(b1, ops, eng.kv, eng.states))[0])
            e3.record()
            torch.cuda.synchronize()
            return e0.elapsed_time(e1), e2.elapsed_time(e3)
        bk = runner.bucket(1)
        bk.fill([dict(tokens=[first], start=args.prompt_len, blocks=blocks, slot=slot)])
        bk.dev.copy_(bk.host, non_blocking=True)
        bk.hist_n.zero_()
        e2.record()
        for _ in range(ticks):
            bk.graph.replay()
        e3.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1), e2.elapsed_time(e3)

    for p in prompts[:W]:
        device_request(p)
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    l0 = native.launch_count
    whole0, whole1 = ev(), ev()
    whole0.record()
    pre_ms, dec_ms = [], []
    for p in prompts[W:]:
        a, b = device_request(p)
        pre_ms.append(a), dec_ms.append(b)
    whole1.record()
    barrier()
    eager_launches = native.launch_count - l0
    graph_kernels = 0 if unfused else runner.bucket(1).kernels
    launches = eager_launches + K * ticks * graph_kernels
    clocks = sampler.stop() if rank == 0 else {}
    for b_ in blocks:
        eng.kv.release(b_)
    eng.states.release(slot)
    t = torch.tensor([sum(pre_ms), sum(dec_ms), whole0.elapsed_time(whole1)], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    pre_total, dec_total, whole_ms = t.tolist()
    decode_tok_s = K * ticks / (dec_total / 1e3)
    prefill_tok_s = K * args.prompt_len / (pre_total / 1e3)

    # ---- end-to-end arm (public engine API) ------------------------------------------------
    for p in prompts[:W]:
        eng.generate([p.tolist()], sp)
    barrier()
    e2e_ms, ttft, e2e_tokens = 0.0, [], 0
    first_tokens = None
    h2d0, d2h0 = eng.io_bytes()
    for p in prompts[W:]:
        a, b = ev(), ev()
        a.record()
        t_host = time.perf_counter()
        # host -> device of this request's prompt ids from pinned memory happens inside the
        # prefill tick (Batch.build); every decode tick copies its input block and reads its token
        res = eng.generate([p.tolist()], sp)[0]
        b.record()
        torch.cuda.synchronize()
        e2e_ms += max(a.elapsed_time(b), (time.perf_counter() - t_host) * 1e3)
        ttft.append(res.ttft_s)
        e2e_tokens += len(res.tokens)
        if first_tokens is None:
            first_tokens = list(res.tokens)
    barrier()
    te = torch.tensor([e2e_ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(te, op=dist.ReduceOp.MAX)
    e2e_ms = float(te[0])
    ttft_ms = statistics.mean(ttft) * 1e3
    e2e_decode_tok_s = K * (args.gen - 1) / max(1e-9, (e2e_ms - K * ttft_ms) / 1e3)
    h2d1, d2h1 = eng.io_bytes()
    h2d, d2h = (h2d1 - h2d0) / K, (d2h1 - d2h0) / K
    err = native.read_error()
    # same-box control at N > 1: this repository's kernels with every collective a library (NCCL) call
    # and eager ticks, one warm-up request and one timed request on the same weights
    value_unfused = None
    if world > 1 and args.impl == "ours" and not args.no_control:
        from tilerl_b200.parallel.symm import NcclComm
        ops_u = make_ops(dev, tp_comm=NcclComm(dist.group.WORLD, dev))
        ops_u.vocab = ops.vocab
        eng_u = build_engine(model, ops_u, slots=2, max_ctx=max_ctx, graph=False, prefix=False)
        blocks_u = [eng_u.kv.alloc_block() for _ in range(nblk)]
        slot_u = eng_u.states.alloc_slot()
        dec_u = 0.0
        for it, p in enumerate(prompts[:2]):
            eng_u.states.states[slot_u].zero_(), eng_u.states.ring[slot_u].zero_()
            eng_u.states.cur[slot_u] = 0
            bu = Batch.build([dict(tokens=p.tolist(), start=0, blocks=blocks_u, slot=slot_u)], dev)
            tk = int(ops_u.argmax(model.forward(bu, ops_u, eng_u.kv, eng_u.states))[0])
            barrier()
            ea, eb = ev(), ev()
            ea.record()
            for i in range(ticks):
                b1 = Batch.build([dict(tokens=[tk], start=args.prompt_len + i, blocks=blocks_u, slot=slot_u)], dev)
                tk = int(ops_u.argmax(model.forward(b1, ops_u, eng_u.kv, eng_u.states))[0])
            eb.record()
            torch.cuda.synchronize()
            dec_u = ea.elapsed_time(eb)
        tu = torch.tensor([dec_u], device=dev, dtype=torch.float64)
        dist.all_reduce(tu, op=dist.ReduceOp.MAX)
        value_unfused = round(ticks / (float(tu[0]) / 1e3), 2)
    if rank == 0:
        out = {
            "impl": args.impl,
            "metric": "decode_tok_s_b1_27b_nvfp4_prompt512_gen64", "value": round(decode_tok_s, 2),
            "unit": "tok/s", "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": round(whole_ms / K, 3), "higher_is_better": True, "scaling": "strong",
            "vs_baseline": round(decode_tok_s / BASELINE_DECODE_TOK_S, 3), "dtype": "nvfp4 weights, bf16 activations",
            "data": "synthetic (uniform-random token ids, random-init N(0,0.02) weights quantised to NVFP4)",
            "config": {"model": cfg.name, "global_batch": 1, "seq_len": args.prompt_len + args.gen,
                       "prompt_len": args.prompt_len, "gen_len": args.gen, "parallelism": f"tp{world}",
                       "l2": ("inputs larger than L2 (every rank holds %.1f GB of weights and streams them each tick)"
                              % (model.served_bytes() / 1e9)),
                       "decode": ("eager ticks, NCCL all-reduce after each row-parallel projection" if unfused
                                  else "CUDA-graph ticks, device-side advance")},
            "prefill_tok_s": round(prefill_tok_s, 1),
            "prefill_vs_baseline": round(prefill_tok_s / BASELINE_PREFILL_TOK_S, 3),
            "decode_ms_per_tick": round(dec_total / (K * ticks), 4),
            "prefill_ms": round(pre_total / K, 3),
            "e2e": {"value": round(e2e_decode_tok_s, 2), "unit": "tok/s (decode, engine API)",
                    "request_ms": round(e2e_ms / K, 3), "ttft_ms": round(ttft_ms, 3),
                    "request_tok_s": round(e2e_tokens / (e2e_ms / 1e3), 2),
                    "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h)},
            "gpu_launches": int(launches), "kernels_per_decode_tick": int(graph_kernels),
            "clocks": clocks, "build_s": round(build_s, 1), "served_bytes": model.served_bytes(),
            "device_error_word": list(err),
            # decode tok/s of the unfused control on the same box and weights (N > 1 only)
            "value_unfused": value_unfused,
            "fused_over_unfused": (round(decode_tok_s / value_unfused, 3) if value_unfused else None),
            # greedy tokens of the first timed request: the same prompt at every GPU count, so runs at
            # N = 1, 2, 4, 8 can be compared (different summation orders may flip a near-tie late on)
            "token_checksum": zlib.crc32(",".join(map(str, first_tokens or [])).encode()),
            "first_tokens": (first_tokens or [])[:16],
        }
        print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
