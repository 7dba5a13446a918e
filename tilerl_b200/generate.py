"""Offline generation, data-parallel by process: one OS process per GPU, a strided slice of
the prompt file each, one output file per worker (no queue, no collective).

Parity: reference ``src/tilerl/generate.py`` -- ``run_worker:26``, ``generate:101``.
"""
from __future__ import annotations

import json
import os
from typing import List, Optional

import torch


def read_prompts(path: str) -> List[str]:
    out = []
    with open(path) as f:
        for ln in f:
            ln = ln.strip()
            if not ln:
                continue
            try:
                j = json.loads(ln)
                out.append(j["prompt"] if isinstance(j, dict) else str(j))
            except json.JSONDecodeError:
                out.append(ln)
    return out


def run_worker(worker: int, n_workers: int, model_name: str, prompts_path: str, out_dir: str, *,
               device: str = "cpu", max_tokens: int = 64, temperature: float = 0.0, checkpoint: Optional[str] = None,
               tokenizer_path: Optional[str] = None, batch: int = 8, seed: int = 0, top_p: float = 1.0,
               top_k: int = 0) -> str:
    from .engine import SamplingParams
    from .factory import build_serving_engine
    from .tokenizer import load_tokenizer
    if device.startswith("cuda"):
        torch.cuda.set_device(worker % max(1, torch.cuda.device_count()))
        device = f"cuda:{worker % max(1, torch.cuda.device_count())}"
    eng = build_serving_engine(model_name, device, checkpoint=checkpoint, slots=batch, max_ctx=4096, seed=seed)
    tok = load_tokenizer(tokenizer_path, eng.model.cfg.vocab)
    prompts = read_prompts(prompts_path)[worker::n_workers]
    os.makedirs(out_dir, exist_ok=True)
    path = os.path.join(out_dir, f"part-{worker:03d}.jsonl")
    with open(path, "w") as f:
        for i in range(0, len(prompts), batch):
            chunk = prompts[i:i + batch]
            ids = [tok.encode(p) for p in chunk]
            sp = [SamplingParams(max_tokens=max_tokens, temperature=temperature, top_p=top_p, top_k=top_k,
                                 seed=seed + worker * 100003 + i + j)
                  for j in range(len(chunk))]
            for p, r in zip(chunk, eng.generate(ids, sp)):
                f.write(json.dumps({"prompt": p, "completion": tok.decode(r.tokens), "tokens": len(r.tokens),
                                    "finish_reason": r.finish_reason}) + "\n")
    return path


def generate(model_name: str, prompts_path: str, out_dir: str, *, workers: int = 1, device: str = "cpu", **kw):
    if workers == 1:
        return [run_worker(0, 1, model_name, prompts_path, out_dir, device=device, **kw)]
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    procs = [ctx.Process(target=run_worker, args=(w, workers, model_name, prompts_path, out_dir),
                         kwargs=dict(device=device, **kw)) for w in range(workers)]
    for p in procs:
        p.start()
    for p in procs:
        p.join()
        if p.exitcode != 0:
            raise RuntimeError(f"generation worker exited with {p.exitcode}")
    return [os.path.join(out_dir, f"part-{w:03d}.jsonl") for w in range(workers)]
