"""Checkpoint merging, streamed tensor by tensor: average, TIES, DARE and iso merges of
fine-tuned checkpoints relative to a base.

Parity: reference ``src/tilerl/merge.py`` (iso / ties / dare / average).
"""
from __future__ import annotations

import os
from typing import Dict, List, Optional, Sequence

import torch


def merge_average(deltas: Sequence[torch.Tensor], weights: Optional[Sequence[float]] = None) -> torch.Tensor:
    w = weights or [1.0 / len(deltas)] * len(deltas)
    return sum(d * wi for d, wi in zip(deltas, w))


def merge_ties(deltas: Sequence[torch.Tensor], density: float = 0.2) -> torch.Tensor:
    """Trim each task vector to its top-``density`` magnitudes, elect a sign per element by
    total mass, and average the entries that agree with it."""
    trimmed = []
    for d in deltas:
        k = max(1, int(d.numel() * density))
        thr = d.abs().flatten().kthvalue(d.numel() - k + 1).values
        trimmed.append(torch.where(d.abs() >= thr, d, torch.zeros_like(d)))
    st = torch.stack(trimmed)
    sign = torch.sign(st.sum(0))
    agree = (torch.sign(st) == sign) & (st != 0)
    return (st * agree).sum(0) / agree.sum(0).clamp_min(1)


def merge_dare(deltas: Sequence[torch.Tensor], drop: float = 0.9, seed: int = 0) -> torch.Tensor:
    """Drop each delta entry with probability ``drop`` and rescale the rest by 1/(1-drop)."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    out = torch.zeros_like(deltas[0])
    for d in deltas:
        keep = (torch.rand(d.shape, generator=g) >= drop).to(d.dtype).to(d.device)
        out += d * keep / (1.0 - drop)
    return out / len(deltas)


def merge_iso(deltas: Sequence[torch.Tensor]) -> torch.Tensor:
    """Isotropic merge: sum the task vectors, then flatten the spectrum of 2-D tensors to its
    mean singular value so no task dominates a direction."""
    s = sum(deltas)
    if s.dim() != 2 or min(s.shape) < 2:
        return s / len(deltas)
    u, sv, vh = torch.linalg.svd(s.float(), full_matrices=False)
    return (u * sv.mean()) @ vh


METHODS = {"average": merge_average, "ties": merge_ties, "dare": merge_dare, "iso": merge_iso}


def merge_checkpoints(base: str, tuned: List[str], out: str, method: str = "average", **kw) -> int:
    """Stream safetensors files: ``out = base + merge(tuned_i - base)`` per tensor."""
    from safetensors import safe_open
    from safetensors.torch import save_file
    fn = METHODS[method]
    f_base = safe_open(os.path.join(base, "model.safetensors"), framework="pt")
    f_tuned = [safe_open(os.path.join(t, "model.safetensors"), framework="pt") for t in tuned]
    result: Dict[str, torch.Tensor] = {}
    for name in f_base.keys():
        b = f_base.get_tensor(name)
        if not b.dtype.is_floating_point or b.dtype == torch.float8_e4m3fn or any(name not in f.keys() for f in f_tuned):
            result[name] = b
            continue
        deltas = [f.get_tensor(name).float() - b.float() for f in f_tuned]
        result[name] = (b.float() + fn(deltas, **kw)).to(b.dtype)
    os.makedirs(out, exist_ok=True)
    save_file(result, os.path.join(out, "model.safetensors"))
    return len(result)
