"""Append-only bench record store with schema validation, a metric registry with physical
floors, and the regression gate.

A record is one JSON line ``{metric, value, unit, target, build, shape, warm, commit, floor,
ts}``.  ``validate`` rejects unknown metrics, wrong units, missing shape keys and values that
beat their physical floor (marked ``IMPLAUSIBLE``); ``gate`` compares a new value against the
stored baseline and fails below 0.97x (or above 1/0.97x for lower-is-better metrics).

Parity: reference ``src/tilerl/benchrec.py`` and ``docs/bench-schema.md:1-80``,
``docs/bench-metrics.json``, ``docs/experience/wins/bench-baseline.json``.
"""
from __future__ import annotations

import json
import os
import subprocess
import time
from typing import Any, Dict, List, Optional

STORE = os.environ.get("TRL_BENCH_STORE", os.path.join("bench", "measurements.jsonl"))


def store_path() -> str:
    return os.environ.get("TRL_BENCH_STORE", STORE)
GATE_RATIO = 0.97

# metric -> (unit, higher_is_better, required shape keys)
METRICS: Dict[str, tuple] = {
    "decode_tok_s": ("tok/s", True, ("model", "batch", "ctx", "tp")),
    "prefill_tok_s": ("tok/s", True, ("model", "prompt_len", "tp")),
    "decode_ms_per_tick": ("ms", False, ("model", "batch", "ctx", "tp")),
    "spec_goodput_tok_s": ("tok/s", True, ("model", "width", "tp")),
    "verify_tick_ms": ("ms", False, ("model", "width", "acceptance", "tp")),
    "sparse_decode_ms_per_tick": ("ms", False, ("model", "ctx", "top_k", "tp")),
    "train_step_tok_s": ("tok/s", True, ("model", "batch", "ctx", "mode")),
    "grpo_step_s": ("s", False, ("model", "group", "prompts", "gen", "gpus")),
    "gemv_gbs": ("GB/s", True, ("n", "k", "m")),
    "gemm_tflops": ("TFLOP/s", True, ("m", "n", "k", "terms")),
    "allreduce_us": ("us", False, ("bytes", "tp")),
    "hbm_copy_gbs": ("GB/s", True, ()),
    "bf16_gemm_tflops": ("TFLOP/s", True, ()),
    "e2e_request_tok_s": ("tok/s", True, ("model", "prompt_len", "gen", "tp")),
    "ttft_ms": ("ms", False, ("model", "prompt_len", "tp")),
    "mmlu_acc": ("frac", True, ("model", "n")),
    "gsm8k_acc": ("frac", True, ("model", "n")),
    "kv_boot_s": ("s", False, ("model", "entries")),
    "resync_ms": ("ms", False, ("model", "tp")),
    # what a serving engine holds after its warm-up: the sum of its static pools and the allocator's peak above it
    "resident_peak_bytes": ("B", False, ("model", "slots", "tp")),
    "resident_static_bytes": ("B", False, ("model", "slots", "tp")),
    "resident_transient_bytes": ("B", False, ("model", "slots", "tp")),
}


class SchemaError(ValueError):
    pass


def _commit() -> str:
    try:
        return subprocess.run(["git", "rev-parse", "--short", "HEAD"], capture_output=True, text=True,
                              timeout=5).stdout.strip() or "unknown"
    except Exception:  # noqa: BLE001
        return "unknown"


def make_record(metric: str, value: float, shape: Dict[str, Any], *, target: str = "b200", build: str = "aot",
                warm: int = 3, floor: Optional[float] = None, commit: Optional[str] = None) -> Dict[str, Any]:
    unit = METRICS.get(metric, ("?",))[0]
    return {"metric": metric, "value": float(value), "unit": unit, "target": target, "build": build,
            "shape": dict(shape), "warm": int(warm), "commit": commit or _commit(), "floor": floor,
            "ts": round(time.time(), 1)}


def validate(rec: Dict[str, Any]) -> Dict[str, Any]:
    for k in ("metric", "value", "unit", "target", "build", "shape", "warm", "commit"):
        if k not in rec:
            raise SchemaError(f"record lacks {k!r}")
    if rec["metric"] not in METRICS:
        raise SchemaError(f"unknown metric {rec['metric']!r}")
    unit, hib, keys = METRICS[rec["metric"]]
    if rec["unit"] != unit:
        raise SchemaError(f"{rec['metric']} is measured in {unit}, got {rec['unit']!r}")
    missing = [k for k in keys if k not in rec["shape"]]
    if missing:
        raise SchemaError(f"shape lacks {missing}")
    if rec["warm"] < 3:
        raise SchemaError("at least 3 warm-up iterations are required")
    if not (rec["value"] == rec["value"]) or rec["value"] <= 0:
        raise SchemaError("value must be a positive number")
    floor = rec.get("floor")
    rec = dict(rec)
    if floor is not None:
        beats = rec["value"] > floor if hib else rec["value"] < floor
        rec["status"] = "IMPLAUSIBLE" if beats else "ok"
    else:
        rec["status"] = "ok"
    return rec


def append(rec: Dict[str, Any], path: Optional[str] = None) -> Dict[str, Any]:
    rec = validate(rec)
    path = path or store_path()
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    with open(path, "a") as f:
        f.write(json.dumps(rec, sort_keys=True) + "\n")
    return rec


def load(path: str = STORE) -> List[Dict[str, Any]]:
    if not os.path.exists(path):
        return []
    with open(path) as f:
        return [json.loads(ln) for ln in f if ln.strip()]


def _same_shape(a: Dict[str, Any], b: Dict[str, Any]) -> bool:
    return a["metric"] == b["metric"] and a["shape"] == b["shape"] and a.get("target") == b.get("target")


def baseline_for(rec: Dict[str, Any], records: List[Dict[str, Any]]) -> Optional[Dict[str, Any]]:
    """Best earlier plausible record of the same metric and shape."""
    hib = METRICS[rec["metric"]][1]
    cands = [r for r in records if _same_shape(r, rec) and r.get("status", "ok") == "ok"]
    if not cands:
        return None
    return max(cands, key=lambda r: r["value"]) if hib else min(cands, key=lambda r: r["value"])


def gate(rec: Dict[str, Any], records: List[Dict[str, Any]], ratio: float = GATE_RATIO) -> Dict[str, Any]:
    base = baseline_for(rec, records)
    if base is None:
        return {"passed": True, "reason": "no baseline", "ratio": None}
    hib = METRICS[rec["metric"]][1]
    r = rec["value"] / base["value"] if hib else base["value"] / rec["value"]
    return {"passed": r >= ratio, "ratio": round(r, 4), "baseline": base["value"], "baseline_commit": base["commit"]}


def records_from_bench_line(line: Dict[str, Any], *, hbm_gbs: Optional[float] = None) -> List[Dict[str, Any]]:
    """The records held by one JSON line of the repository's ``bench.py`` (decode and prefill
    throughput, tick time, end-to-end request rate, time to first token), with the decode floor
    from the served bytes a tick streams at ``hbm_gbs`` (no floor without it)."""
    cfg = line.get("config", {})
    tp = int(line.get("n_gpus", 1))
    model, plen, gen = cfg.get("model", "?"), int(cfg.get("prompt_len", 0)), int(cfg.get("gen_len", 0))
    warm = int(line.get("warmup", 3))
    floor_tok_s = None
    if hbm_gbs and line.get("served_bytes"):
        floor_tok_s = hbm_gbs * 1e9 / float(line["served_bytes"])     # a tick cannot stream faster than HBM
    dshape = {"model": model, "batch": 1, "ctx": plen, "tp": tp}
    out = [make_record("decode_tok_s", line["value"], dshape, warm=warm, floor=floor_tok_s)]
    if line.get("decode_ms_per_tick"):
        out.append(make_record("decode_ms_per_tick", line["decode_ms_per_tick"], dshape, warm=warm,
                               floor=(1e3 / floor_tok_s if floor_tok_s else None)))
    if line.get("prefill_tok_s"):
        out.append(make_record("prefill_tok_s", line["prefill_tok_s"], {"model": model, "prompt_len": plen, "tp": tp},
                               warm=warm))
    e2e = line.get("e2e") or {}
    if e2e.get("request_tok_s"):
        out.append(make_record("e2e_request_tok_s", e2e["request_tok_s"],
                               {"model": model, "prompt_len": plen, "gen": gen, "tp": tp}, warm=warm))
    if e2e.get("ttft_ms"):
        out.append(make_record("ttft_ms", e2e["ttft_ms"], {"model": model, "prompt_len": plen, "tp": tp}, warm=warm))
    return out
