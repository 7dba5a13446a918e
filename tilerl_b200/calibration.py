"""Measured floors of the machine the engine runs on: HBM copy bandwidth, host-to-device
bandwidth, bf16 library GEMM throughput, and (with >1 GPU) peer copy bandwidth.

``load_peaks`` prefers the driver-written ``MEASURED_PEAKS.json`` at the repository root,
then a previous calibration file, then the fallback figures (6.65 TB/s, 1.59 PFLOP/s).
``calibrate`` measures them with CUDA events (3 warm-ups, best of N).

Parity: reference ``src/tilerl/calibration.py:147,202,215,229,253,326,481``.
"""
from __future__ import annotations

import json
import os
from dataclasses import asdict, dataclass
from typing import Optional

FALLBACK = dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, nvlink_gbs=770.0,
                source="fallback")
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@dataclass
class Peaks:
    hbm_gbs: float
    bf16_tflops: float
    bf16_tflops_sustained: float
    nvlink_gbs: float = 770.0
    h2d_gbs: float = 0.0
    source: str = "measured"


def load_peaks(path: Optional[str] = None) -> Peaks:
    for p in (path, os.path.join(ROOT, "MEASURED_PEAKS.json"), os.path.join(ROOT, "calibration.json")):
        if p and os.path.exists(p):
            with open(p) as f:
                d = json.load(f)
            return Peaks(float(d["hbm_gbs"]), float(d["bf16_tflops"]),
                         float(d.get("bf16_tflops_sustained", d["bf16_tflops"])),
                         float(d.get("nvlink_gbs", 770.0)), float(d.get("h2d_gbs", 0.0)), "measured")
    return Peaks(**FALLBACK)


# Floors of other parts, for reading the declared cost table against the hardware a published figure was
# taken on.  These are the vendors' nominal dense figures (memory GB/s, bf16 or fp16 tensor TFLOP/s, link
# GB/s per direction), not measurements; only the B200 row is measured (or the pool's earlier fallback).
NOMINAL = {
    "h20": dict(hbm_gbs=4000.0, bf16_tflops=148.0, bf16_tflops_sustained=148.0, nvlink_gbs=450.0, source="nominal"),
    "h100": dict(hbm_gbs=3350.0, bf16_tflops=989.0, bf16_tflops_sustained=989.0, nvlink_gbs=450.0, source="nominal"),
    "v100": dict(hbm_gbs=900.0, bf16_tflops=125.0, bf16_tflops_sustained=125.0, nvlink_gbs=150.0, source="nominal"),
}


def peaks_for(device_name: Optional[str] = None, path: Optional[str] = None) -> Peaks:
    """Floors the cost table is divided by: ``None`` / ``b200`` -> this machine's measured file (or the
    fallback); another known name -> its nominal figures; an unknown name has no floor (reference
    ``tilerl bench --kernels --device-name``, ``src/tilerl/calibration.py``)."""
    name = (device_name or "b200").lower().replace("nvidia", "").replace("-", "").replace(" ", "")
    if name.startswith("b200"):
        return load_peaks(path)
    for key, row in NOMINAL.items():
        if name.startswith(key):
            return Peaks(**row)
    raise KeyError(f"no floor known for device {device_name!r}; known: b200, {', '.join(sorted(NOMINAL))}")


def _best_ms(fn, reps: int = 10, warm: int = 3) -> float:
    import torch
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    best = float("inf")
    for _ in range(reps):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        best = min(best, a.elapsed_time(b))
    return best


def calibrate(device="cuda", elems: int = 1 << 29, out: Optional[str] = None) -> Peaks:
    import torch
    dev = torch.device(device)
    a = torch.empty(elems, dtype=torch.bfloat16, device=dev)
    b = torch.empty_like(a)
    hbm = 2 * a.numel() * 2 / (_best_ms(lambda: b.copy_(a)) * 1e-3) / 1e9
    n = 8192
    x = torch.randn(n, n, device=dev, dtype=torch.bfloat16)
    y = torch.randn(n, n, device=dev, dtype=torch.bfloat16)
    tf = 2.0 * n ** 3 / (_best_ms(lambda: torch.matmul(x, y)) * 1e-3) / 1e12
    host = torch.empty(1 << 28, dtype=torch.uint8).pin_memory()
    dst = torch.empty(1 << 28, dtype=torch.uint8, device=dev)
    h2d = host.numel() / (_best_ms(lambda: dst.copy_(host, non_blocking=True)) * 1e-3) / 1e9
    link = 770.0
    if torch.cuda.device_count() > 1:
        peer = torch.empty(1 << 28, dtype=torch.uint8, device="cuda:1")
        link = dst.numel() / (_best_ms(lambda: peer.copy_(dst)) * 1e-3) / 1e9
    p = Peaks(hbm, tf, tf, link, h2d, "measured")
    if out:
        with open(out, "w") as f:
            json.dump(asdict(p), f, indent=1)
    return p
