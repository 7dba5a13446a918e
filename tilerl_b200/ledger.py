"""Run ledger: every training / eval run gets ``runs/<id>/manifest.json`` whose id is a hash
of its inputs (flags, model, data, parent run), with gates, lineage and early stopping.

Parity: reference ``src/tilerl/ledger.py:245,299,549`` (manifest, gates, ``EarlyStop``,
``time_to_score``, ``ledger --devices``).
"""
from __future__ import annotations

import hashlib
import json
import os
import time
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

def runs_dir() -> str:
    """Where run manifests live: ``$TRL_RUNS`` (read at call time, so a test or a job can point it
    elsewhere) or ``./runs``."""
    return os.environ.get("TRL_RUNS", "runs")



def run_id(inputs: Dict[str, Any]) -> str:
    blob = json.dumps(inputs, sort_keys=True, default=str).encode()
    return hashlib.sha256(blob).hexdigest()[:12]


@dataclass
class Gate:
    name: str
    value: float
    threshold: float
    higher_is_better: bool = True

    @property
    def passed(self) -> bool:
        return self.value >= self.threshold if self.higher_is_better else self.value <= self.threshold


@dataclass
class Run:
    inputs: Dict[str, Any]
    root: str = field(default_factory=runs_dir)
    parent: Optional[str] = None
    id: str = ""
    metrics: List[Dict[str, Any]] = field(default_factory=list)
    gates: List[Gate] = field(default_factory=list)
    artifacts: Dict[str, str] = field(default_factory=dict)
    started: float = field(default_factory=time.time)
    status: str = "running"
    parents: List[str] = field(default_factory=list)     # a merge descends from the runs that wrote its inputs

    def __post_init__(self):
        self.id = self.id or run_id({**self.inputs, "parent": self.parent})
        os.makedirs(self.dir, exist_ok=True)
        self.write()

    @property
    def dir(self) -> str:
        return os.path.join(self.root, self.id)

    def log(self, **m) -> None:
        self.metrics.append({"t": round(time.time() - self.started, 3), **m})

    def gate(self, name: str, value: float, threshold: float, higher_is_better: bool = True) -> bool:
        g = Gate(name, float(value), float(threshold), higher_is_better)
        self.gates.append(g)
        return g.passed

    def finish(self, status: str = "done") -> None:
        self.status = status if all(g.passed for g in self.gates) else "gate_failed"
        self.write()

    def write(self) -> None:
        man = {"id": self.id, "parent": self.parent, "inputs": self.inputs, "status": self.status,
               "parents": list(self.parents), "started": self.started, "seconds": round(time.time() - self.started, 3), "metrics": self.metrics,
               "gates": [{"name": g.name, "value": g.value, "threshold": g.threshold, "passed": g.passed}
                         for g in self.gates], "artifacts": self.artifacts}
        tmp = os.path.join(self.dir, "manifest.json.tmp")
        with open(tmp, "w") as f:
            json.dump(man, f, indent=1, default=str)
        os.replace(tmp, os.path.join(self.dir, "manifest.json"))


def finished_run(inputs: Dict[str, Any], parent: Optional[str] = None, root: Optional[str] = None
                 ) -> Optional[Dict[str, Any]]:
    """The manifest of a run with exactly these inputs that already ended with status ``done``, else None.
    A run's id is the hash of its inputs, so the same command asked twice is the same run: the caller
    hands back the finished manifest instead of training again unless it was told to (``train --force``;
    reference ``src/tilerl/ledger.py`` finish / reuse of a finished manifest)."""
    try:
        man = load_run(run_id({**inputs, "parent": parent}), root)
    except (OSError, json.JSONDecodeError):
        return None
    return man if man.get("status") == "done" else None


def find_run_for_artifact(path: str, root: Optional[str] = None) -> Optional[str]:
    """Id of the newest finished run whose manifest lists ``path`` among its artifacts, else None.  A
    checkpoint directory carries no run id of its own; lineage goes through the manifest that wrote it, and
    an id is never guessed from a path component.  Reference ``src/tilerl/cli.py:386-392``."""
    want = os.path.realpath(path)
    best = None
    for man in list_runs(root):
        if man.get("status") != "done":
            continue
        if any(os.path.realpath(str(v)) == want for v in (man.get("artifacts") or {}).values()):
            if best is None or man.get("started", 0) >= best.get("started", 0):
                best = man
    return best["id"] if best else None


def load_run(rid: str, root: Optional[str] = None) -> Dict[str, Any]:
    with open(os.path.join(root or runs_dir(), rid, "manifest.json")) as f:
        return json.load(f)


def lineage(rid: str, root: Optional[str] = None) -> List[str]:
    chain = []
    cur: Optional[str] = rid
    while cur and cur not in chain:
        chain.append(cur)
        try:
            cur = load_run(cur, root).get("parent")
        except OSError:
            break
    return chain


def list_runs(root: Optional[str] = None) -> List[Dict[str, Any]]:
    out = []
    root = root or runs_dir()
    if os.path.isdir(root):
        for d in sorted(os.listdir(root)):
            try:
                out.append(load_run(d, root))
            except (OSError, json.JSONDecodeError):
                continue
    return out


def time_to_score(run: Dict[str, Any], key: str, target: float) -> Optional[float]:
    for m in run.get("metrics", []):
        if key in m and m[key] >= target:
            return m["t"]
    return None


def refuse_blind_curve(n: int, target_pt: float) -> None:
    """Refuse an accuracy curve whose subset cannot resolve the effect it is there to locate, before the
    run spends the time.  Worst-case binomial standard error (p = 0.5) in points is 50 / sqrt(n); strictly
    above the target, the step at which the curve crosses would be chosen by which rows fell into the
    subset.  Reference ``src/tilerl/ledger.py:614``."""
    if n <= 0:
        return
    se = 50.0 / (n ** 0.5)
    if se > target_pt:
        raise SystemExit(f"--eval-curve-n {n} carries a worst-case binomial SE of {se:.1f} pt, above the "
                         f"--curve-target-pt {target_pt:g} effect the curve locates: the crossing step would be chosen "
                         f"by which rows fell where. Raise --eval-curve-n to >={(50.0 / target_pt) ** 2:.0f}, or raise "
                         f"the target")


def curve_rows(rows: List[Any], n: int, seed: int) -> List[Any]:
    """The curve subset: the first ``n`` rows of a fixed-seed shuffle, not of the file (an ordered test file
    biases its head), the same rows at every step and in every run so that points pair up.  Reference
    ``src/tilerl/train.py:1729``."""
    import random
    pool = list(rows)
    random.Random(seed).shuffle(pool)
    return pool[:n]


def binomial_se_pt(correct_rate: float, n: int) -> float:
    """Standard error of an accuracy measured on ``n`` rows, in points, at the point's own rate."""
    return 100.0 * (max(0.0, correct_rate * (1.0 - correct_rate)) / max(1, n)) ** 0.5


class EarlyStop:
    """Stop when the monitored score has not improved by ``min_delta`` for ``patience`` evals."""

    def __init__(self, patience: int = 3, min_delta: float = 0.0):
        self.patience, self.min_delta = patience, min_delta
        self.best: Optional[float] = None
        self.best_step = -1
        self.bad = 0

    def update(self, score: float, step: int) -> bool:
        """Returns True when training should stop; ``improved`` tells whether to save."""
        self.improved = self.best is None or score > self.best + self.min_delta
        if self.improved:
            self.best, self.best_step, self.bad = score, step, 0
        else:
            self.bad += 1
        return self.bad >= self.patience


def devices() -> List[Dict[str, Any]]:
    """What ``ledger --devices`` prints: one row per visible GPU (read-only queries)."""
    try:
        import torch
        return [{"index": i, "name": torch.cuda.get_device_name(i),
                 "total_gib": round(torch.cuda.get_device_properties(i).total_memory / 2 ** 30, 1),
                 "sms": torch.cuda.get_device_properties(i).multi_processor_count}
                for i in range(torch.cuda.device_count())]
    except Exception:  # noqa: BLE001
        return []


def device_sections(records: List[Dict[str, Any]]) -> List[Dict[str, Any]]:
    """One section per target in the bench store: its newest measured floors (copy bandwidth, bf16 GEMM
    rate) and its newest residency triple.  Reference ``src/tilerl/cli.py`` (``_device_ledger_rows``)."""
    out: Dict[str, Dict[str, Any]] = {}
    for r in sorted(records, key=lambda r: r.get("ts", 0)):
        sec = out.setdefault(r.get("target", "?"), {"device": r.get("target", "?"), "hbm_copy_gbs": None,
                                                    "bf16_gemm_tflops": None, "residency": None})
        m = r.get("metric")
        if m in ("hbm_copy_gbs", "bf16_gemm_tflops"):
            sec[m] = {"value": r["value"], "commit": r.get("commit"), "ts": r.get("ts")}
        elif m in ("resident_peak_bytes", "resident_static_bytes", "resident_transient_bytes"):
            res = sec["residency"] if sec["residency"] and sec["residency"].get("shape") == r.get("shape") else \
                {"shape": r.get("shape"), "commit": r.get("commit"), "ts": r.get("ts")}
            res[m.split("_")[1]] = r["value"]
            sec["residency"] = res
    return list(out.values())


def format_device_sections(sections: List[Dict[str, Any]]) -> str:
    lines = ["devices (newest measured floor + residency per target):"]
    for s in sections:
        lines.append(f"  {s['device']}")
        bw, pk, res = s["hbm_copy_gbs"], s["bf16_gemm_tflops"], s["residency"]
        if bw is None or pk is None:
            lines.append("    copy bandwidth / bf16 peak: none recorded (run bench --calibrate --record)")
        else:
            lines.append(f"    hbm_copy_gbs {bw['value']:.1f} (commit {bw['commit']})  bf16_gemm_tflops {pk['value']:.1f} "
                         f"(commit {pk['commit']})")
        if res is None or "peak" not in res:
            lines.append("    residency: none recorded (run serve --record-residency)")
        else:
            mib = 2 ** 20
            lines.append(f"    resident {res['peak'] / mib:10.2f} MiB = static {res.get('static', 0) / mib:.2f} + transient "
                         f"{res.get('transient', 0) / mib:.2f}  {res['shape']} (commit {res['commit']})")
    if len(lines) == 1:
        lines.append("  (no calibration or residency rows in the bench store)")
    return "\n".join(lines)
