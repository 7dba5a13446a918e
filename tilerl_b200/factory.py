"""Wiring: build a model, size its pools, assemble an engine.

``build_model`` creates the (optionally TP-sharded) served parameters either from
a checkpoint directory or from a seeded random initialisation.  Random weights
are generated tensor by tensor directly on the target device and quantised
there, so the 27B never exists in full precision anywhere (its fp32 master
would be 108 GB).  ``fit_blocks`` derives the KV page count from free device
memory; ``build_engine`` creates pools, prefix store, CUDA-graph runner and the
engine.

Parity: reference ``src/tilerl/build.py`` -- ``build_model:76``, ``_shard:46``,
``fit_blocks:118``, ``build_engine:151-579``, ``build_serving_engine:582``.
"""
from __future__ import annotations

import zlib
from typing import Dict, Optional

import torch

from .config import ModelConfig, get_config
from .engine import Engine, StepLimits
from .formats import NVFP4Tensor
from .kv import GdnStatePool, NoPrefixStore, PagedKvPool, PrefixStore
from .models.hybrid import HybridModel, linear_names, param_shapes, quantize_weight
from .ops.backend import RefOps
from .ops.ref import KV_BLOCK


def _seed_for(name: str, seed: int) -> int:
    return (zlib.crc32(name.encode()) ^ (seed * 0x9E3779B1)) & 0x7FFFFFFF


def random_param(cfg: ModelConfig, name: str, shape, seed: int, device) -> torch.Tensor:
    """One full (unsharded) parameter, deterministic in (name, seed) on any rank."""
    g = torch.Generator(device=device).manual_seed(_seed_for(name, seed))
    leaf = name.split(".")[-1]
    if leaf in ("norm1", "norm2", "final_norm", "q_norm", "k_norm", "gdn_norm"):
        return torch.ones(shape, device=device)
    if leaf == "a_log":
        return torch.log(torch.empty(shape, device=device).uniform_(1.0, 16.0, generator=g))
    if leaf == "dt_bias":
        return torch.empty(shape, device=device).uniform_(-1.0, 1.0, generator=g)
    if leaf == "conv":
        return torch.randn(shape, device=device, generator=g) * 0.3
    return torch.randn(shape, device=device, generator=g, dtype=torch.float32) * 0.02


def build_random_streaming(cfg: ModelConfig, device, seed: int = 0, tp_rank: int = 0, tp: int = 1,
                           ops=None, keep_master: bool = False, master_only: bool = False) -> HybridModel:
    """``master_only``: a trainer that never serves keeps just the master projections (no
    quantised copy is built)."""
    from .parallel.mesh import shard_param
    device = torch.device(device)
    lin = set(linear_names(cfg))
    params: Dict[str, object] = {}
    for name, shape in param_shapes(cfg, 1).items():
        full = random_param(cfg, name, shape, seed, device)
        w = shard_param(cfg, name, full, tp_rank, tp)
        if master_only and name in lin:
            params["master." + name] = w.to(torch.bfloat16) if device.type == "cuda" else w.clone()
        elif name in lin or (name == "lm_head" and cfg.lm_head_quant == "nvfp4"):
            if cfg.quant == "nvfp4" and device.type == "cuda" and ops is not None:
                # quantise the full tensor on the device, then cut the packed planes
                n, k = full.shape
                q = NVFP4Tensor(torch.empty(n, k // 2, dtype=torch.uint8, device=device),
                                torch.empty(n, k // 16, dtype=torch.float8_e4m3fn, device=device),
                                torch.empty(1, dtype=torch.float32, device=device))
                ops.quantize_nvfp4_(full.contiguous(), q)
                params[name] = shard_param(cfg, name, q, tp_rank, tp)
            elif cfg.quant == "nvfp4":
                params[name] = shard_param(cfg, name, quantize_weight(full.float(), "nvfp4"), tp_rank, tp)
            else:
                params[name] = quantize_weight(w.float(), cfg.quant)
            if keep_master:
                params["master." + name] = w.to(torch.bfloat16) if device.type == "cuda" else w.clone()
        elif name in ("embed", "lm_head"):
            params[name] = w.to(torch.bfloat16 if device.type == "cuda" else torch.float32)
        else:
            params[name] = w.float()
        del w, full
    if device.type == "cuda":
        torch.cuda.synchronize()
    return HybridModel(cfg, params, tp_rank, tp)


def materialize(model: HybridModel, ops) -> None:
    """Create the device-side operand layouts up front (tile-contiguous weight nibbles and
    128x4-tiled scales for the tcgen05 GEMM, the stream layout of the decode GEMV) so the first
    request does not pay for them.
    Reference: ``Backend.materialize`` (``backend.py:975-1021``)."""
    if getattr(ops, "name", "") != "cuda" or not getattr(ops, "use_tc_gemm", False):
        return
    from .ops.gemm_tc import sf_tiled, stream_ok, w_stream, wq_tiled
    for v in model.params.values():
        if isinstance(v, NVFP4Tensor):
            sf_tiled(v)
            wq_tiled(v)
            if getattr(ops, "gemv_stream", False) and stream_ok(v):
                w_stream(v)


def build_model(model: str | ModelConfig, device="cpu", *, seed: int = 0, checkpoint: Optional[str] = None,
                tp_rank: int = 0, tp: int = 1, ops=None, keep_master: bool = False,
                master_only: bool = False) -> HybridModel:
    cfg = get_config(model) if isinstance(model, str) else model
    if checkpoint:
        from .checkpoint import load_checkpoint
        return load_checkpoint(cfg, checkpoint, device=device, tp_rank=tp_rank, tp=tp, keep_master=keep_master)
    m = build_random_streaming(cfg, device, seed, tp_rank, tp, ops, keep_master, master_only)
    if ops is not None and not master_only:
        materialize(m, ops)
    return m


def fit_blocks(cfg: ModelConfig, free_bytes: int, slots: int, *, planes: int = 1, tp: int = 1,
               pool_fraction: float = 2.0 / 3.0, max_blocks: int = 1 << 20, kv_fp8: bool = False) -> int:
    """KV pages that fit in ``pool_fraction`` of what is left after the GDN state slots."""
    from .parallel.mesh import tp_dims
    d = tp_dims(cfg, tp)
    gd = cfg.gdn_head_dim
    slot_bytes = cfg.n_gdn_layers * (planes * d.gdn_nv * gd * gd * 4 + 16 * d.gdn_conv_dim * 2)
    left = free_bytes - slots * slot_bytes
    per_block = max(1, cfg.n_attn_layers) * d.n_kv * KV_BLOCK * cfg.head_dim * 2 * 2
    if kv_fp8:   # one byte per value plus one fp32 scale per (token, head), K and V
        per_block = max(1, cfg.n_attn_layers) * d.n_kv * KV_BLOCK * (cfg.head_dim + 4) * 2
    return int(max(2, min(max_blocks, left * pool_fraction // per_block)))


def make_ops(device, tp_comm=None):
    device = torch.device(device)
    if device.type == "cuda":
        from .ops.cuda import CudaOps
        return CudaOps(device, comm=tp_comm)
    return RefOps()


def build_engine(model: HybridModel, ops=None, *, device=None, blocks: Optional[int] = None, slots: int = 8,
                 max_ctx: int = 4096, prefix: bool = True, graph: bool = True, spec_width: int = 0,
                 drafter=None, limits: Optional[StepLimits] = None, sparse=None, kv_fp8: bool = False,
                 reserve_bytes: int = 0, **engine_kw) -> Engine:
    cfg = model.cfg
    if device is None:
        e = model.params["embed"]
        device = e.device
    device = torch.device(device)
    ops = ops or make_ops(device)
    if hasattr(ops, "vocab"):
        ops.vocab = cfg.vocab
    planes = max(1, spec_width)
    d = model.dims
    if blocks is None:
        if device.type == "cuda":
            free, _ = torch.cuda.mem_get_info(device)
            free = max(0, free - int(reserve_bytes))
            blocks = fit_blocks(cfg, free, slots, planes=planes, tp=model.tp, kv_fp8=kv_fp8,
                                max_blocks=slots * ((max_ctx + KV_BLOCK - 1) // KV_BLOCK) + 2)
        else:
            blocks = slots * ((max_ctx + KV_BLOCK - 1) // KV_BLOCK) + 2
    on_gpu = device.type == "cuda"
    if kv_fp8 and sparse is not None and on_gpu:
        raise ValueError("sparse page selection reads a bf16 KV pool on the device: use --kv-format bf16 with --sparse-k")
    kv = PagedKvPool(cfg, blocks, device, dtype=torch.bfloat16 if on_gpu else torch.float32, n_kv_heads=d.n_kv,
                     fp8=kv_fp8)
    st = GdnStatePool(cfg, slots + 1, device, planes=planes,
                      ring_dtype=torch.bfloat16 if on_gpu else torch.float32,
                      n_v_heads=d.gdn_nv or None, n_k_heads=d.gdn_nk or None)
    runner = vrunner = None
    if graph and on_gpu:
        from .graph import DecodeGraphRunner, VerifyGraphRunner
        runner = DecodeGraphRunner(model, ops, kv, st, max_ctx=max_ctx)
        if spec_width > 0 and drafter is not None:
            vrunner = VerifyGraphRunner(model, ops, kv, st, max_ctx=max_ctx, width=spec_width,
                                        aux_layers=tuple(getattr(drafter, "aux_layers", ())))
    store = PrefixStore(kv) if prefix else NoPrefixStore()
    return Engine(model, ops, kv, st, limits=limits, prefix_store=store, graph_runner=runner,
                  verify_graph_runner=vrunner, drafter=drafter, spec_width=spec_width, sparse=sparse, **engine_kw)


def build_serving_engine(model_name: str = "tiny", device="cpu", **kw) -> Engine:
    ops = make_ops(device)
    seed = kw.pop("seed", 0)
    ckpt = kw.pop("checkpoint", None)
    model = build_model(model_name, device, seed=seed, checkpoint=ckpt, ops=ops if torch.device(device).type == "cuda" else None)
    return build_engine(model, ops, device=device, **kw)
