"""Trainer -> rollout weight resync: after an optimizer step on ZeRO-3 shards, rebuild the
NVFP4 tensor-parallel rollout weights *in place*.

Per unit (decoder layer): gather the full working weights from the shards (the same
all-gather the forward uses), quantise every projection as a FULL tensor (e2m1 + e4m3 per 16 +
fp32 tensor scale -- so all TP ranks serve the values a single-GPU quantisation would),
cut this rank's packed planes and ``copy_`` them into the tensors the rollout engine already
holds: device addresses stay fixed, so captured CUDA graphs and the tile-contiguous copies
the GEMM reads keep working after ``refresh`` re-tiles them.  Vectors (norms, GDN gates) are
copied as they are.  Units are processed one at a time, so at most one layer exists in full
precision; on CUDA the next unit's gather is prefetched while this one is quantised.

Parity: the reference re-packs master -> fp4 in place on one GPU (``requantize_fp4``,
``src/tilerl/model.py:1255-1296``; format maths ``tilerl_kernels/reference.py:299-327``); the
sharded gather and the TP cut are new here.
"""
from __future__ import annotations

import time
from typing import Callable, Dict, Optional

import torch

from ..formats import NVFP4Tensor, quantize_nvfp4
from ..models.hybrid import linear_names
from .mesh import shard_param


def _store(dst, src) -> int:
    """In-place update of one served parameter; returns bytes written."""
    if isinstance(dst, NVFP4Tensor):
        dst.wq.copy_(src.wq)
        dst.scale.copy_(src.scale)
        dst.tscale.copy_(src.tscale)
        return dst.wq.numel() + dst.scale.numel() + 4
    dst.copy_(src.to(dst.dtype))
    return dst.numel() * dst.element_size()


def resync(zero, rollout, *, quantize: Optional[Callable] = None, refresh: Optional[Callable] = None,
           engine=None) -> Dict[str, float]:
    """Write the trainer's current weights into ``rollout`` (a served ``HybridModel`` of TP
    degree ``rollout.tp``).  ``quantize(w_full) -> NVFP4Tensor`` defaults to the torch
    quantiser (a CUDA backend passes its kernel); ``refresh(param)`` is called for every
    rewritten quantised tensor (the CUDA backend re-tiles its GEMM copies there)."""
    cfg = rollout.cfg
    quantize = quantize or (lambda w: quantize_nvfp4(w.float()))
    lin = set(linear_names(cfg))
    t0 = time.perf_counter()
    nbytes = 0
    n_units = len(zero.units)
    with torch.no_grad():
        for i in range(n_units):
            tensors = zero.unit_tensors(i)
            if i + 1 < n_units:
                zero._prefetch(i + 1)
            for name, w in tensors.items():
                base = name[len("master."):] if name.startswith("master.") else name
                dst = rollout.params.get(base)
                if dst is None:
                    continue
                if base in lin and isinstance(dst, NVFP4Tensor):
                    q = shard_param(cfg, base, quantize(w), rollout.tp_rank, rollout.tp)
                    nbytes += _store(dst, q)
                    if refresh is not None:
                        refresh(dst)
                else:
                    src = shard_param(cfg, base, w, rollout.tp_rank, rollout.tp)
                    nbytes += _store(dst, src)
            zero._drop(zero.units[i])
    rollout.weights_version += 1
    if engine is not None:
        engine.invalidate_weights()
    if zero.device.type == "cuda":
        torch.cuda.synchronize(zero.device)
    return dict(seconds=time.perf_counter() - t0, bytes=float(nbytes), units=float(n_units))
