"""Memory planner: what fits on a 180 GB B200 (per TP rank) and how the rest is split.

``plan`` prices the served weights (from the format registry), the GDN state slots, the
workspace, and hands ``pool_fraction`` of what remains to the paged KV pool and
``state_fraction`` to the prefix-state store; ``train_plan`` prices adapter / master /
optimizer / gradient / tape bytes for LoRA and ZeRO-3 full-parameter training.
``memory_table`` prints derived vs measured rows with ``transient = peak - sum(static)``;
``measure`` fills the measured column from a live engine's tensors (``held storage``), so a plan can
be checked against what the process really holds.  Optional rows: a block drafter (parameters and the
per-request context K / V), a learned page indexer, the host KV tier; optimizer state for AdamW,
Adafactor (factored second moment) and the ISO frames.

Parity: reference ``src/tilerl/memory.py:24,48,114,215,245,335-378,411,435,542,625,680``.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional

from .config import ModelConfig
from .formats import nbytes, weight_specs
from .parallel.mesh import is_sharded, tp_dims

GIB = 1 << 30
B200_BYTES = 180 * 10 ** 9


@dataclass
class Plan:
    rows: Dict[str, int] = field(default_factory=dict)
    blocks: int = 0
    slots: int = 0
    notes: List[str] = field(default_factory=list)

    @property
    def total(self) -> int:
        return sum(self.rows.values())


def weight_bytes(cfg: ModelConfig, tp: int = 1, tiled_copy: bool = True) -> int:
    total = 0
    for name, (shape, fmt) in weight_specs(cfg).items():
        b = nbytes(fmt, shape)
        if tp > 1 and is_sharded(name):
            b //= tp
        if fmt == "nvfp4" and tiled_copy:
            b *= 3      # tile-contiguous GEMM operand copy and the GEMV stream-layout copy next to the checkpoint layout
        total += b
    return total


def kv_block_bytes(cfg: ModelConfig, tp: int = 1, fp8: bool = False) -> int:
    d = tp_dims(cfg, tp)
    per = d.n_kv * 16 * cfg.head_dim * (1 if fp8 else 2) * 2
    if fp8:
        per += d.n_kv * 16 * 4 * 2
    return per * max(1, cfg.n_attn_layers)


def state_slot_bytes(cfg: ModelConfig, tp: int = 1, planes: int = 1) -> int:
    d = tp_dims(cfg, tp)
    gd = cfg.gdn_head_dim
    return cfg.n_gdn_layers * (planes * d.gdn_nv * gd * gd * 4 + 16 * d.gdn_conv_dim * 2)


def fit_num_blocks(free_bytes: int, per_block: int, fraction: float = 1.0) -> int:
    """Pages of ``per_block`` bytes that fit into ``fraction`` of ``free_bytes`` (0 when nothing is left)."""
    return max(0, int(free_bytes * fraction) // max(1, per_block))


def drafter_bytes(cfg: ModelConfig, *, width: int = 8, n_layers: int = 2, n_heads: int = 8, n_kv_heads: int = 2,
                  taps: int = 3, window: int = 64, ffn_mult: float = 2.0, sel_rank: int = 16, conv_taps: int = 2,
                  conv_group: int = 64, slots: int = 64, itemsize: int = 4) -> Dict[str, int]:
    """Block drafter (``spec.BlockDrafter``): parameter bytes and the context K / V that every running
    request keeps (``window`` rows per layer)."""
    h, hd = cfg.hidden, cfg.hidden // n_heads
    ffn, groups = int(h * ffn_mult), max(1, h // conv_group)
    per_layer = 2 * h + n_heads * hd * h + 2 * n_kv_heads * hd * h + h * n_heads * hd + 2 * ffn * h + h * ffn \
        + 2 * (2 * conv_taps * h + 2 * conv_taps * groups * h)
    params = taps * h * h + h + width * h + 2 * h + n_layers * per_layer + sel_rank * h + 2 * cfg.vocab * sel_rank
    ctx = slots * n_layers * window * 2 * n_kv_heads * hd + slots * window * h
    return {"drafter parameters": params * itemsize, "drafter context (per-request K / V)": ctx * itemsize}


def indexer_bytes(cfg: ModelConfig, *, heads: int = 4, dim: int = 128, tp: int = 1, itemsize: int = 4) -> int:
    """Learned page indexer (``sparse_index.LearnedIndexer``): two projections per attention layer."""
    d = tp_dims(cfg, tp)
    return max(1, cfg.n_attn_layers) * (d.n_q + d.n_kv) * cfg.head_dim * heads * dim * itemsize


def plan(cfg: ModelConfig, *, device_bytes: int = B200_BYTES, tp: int = 1, slots: int = 64, planes: int = 1,
         max_batched_tokens: int = 8192, reserve_bytes: int = 2 * GIB, pool_fraction: float = 2 / 3,
         state_fraction: float = 1 / 4, kv_fp8: bool = False, blocks: Optional[int] = None,
         drafter: Optional[dict] = None, indexer: Optional[dict] = None, host_pages: int = 0,
         state_bytes: int = 0) -> Plan:
    """``drafter`` / ``indexer``: keyword dicts for :func:`drafter_bytes` / :func:`indexer_bytes` (``{}`` for the
    defaults); ``host_pages``: pages of the host KV tier (pinned host memory, reported in the notes, not
    charged to the device); ``state_bytes``: a fixed budget for the prefix store's GDN snapshots (0: the
    default share of what the pool leaves)."""
    p = Plan(slots=slots)
    p.rows["weights"] = weight_bytes(cfg, tp)
    p.rows["gdn state slots"] = slots * state_slot_bytes(cfg, tp, planes)
    if drafter is not None:
        p.rows.update(drafter_bytes(cfg, slots=slots, **drafter))
    if indexer is not None:
        p.rows["page indexer"] = indexer_bytes(cfg, tp=tp, **indexer)
    if host_pages:
        p.notes.append(f"host KV tier: {host_pages * kv_block_bytes(cfg, tp, kv_fp8) / GIB:.2f} GiB of pinned host memory "
                       f"for {host_pages:,} pages")
    d = tp_dims(cfg, tp)
    widest = max(d.qkv_rows, d.gdn_in_rows, 2 * d.ffn)
    p.rows["workspace"] = max_batched_tokens * (widest * 2 + cfg.hidden * 8 + d.ffn * 2) + d.vocab_local * 4 * 64
    p.rows["reserve"] = reserve_bytes
    left = device_bytes - p.total
    if left <= 0:
        p.notes.append("model does not fit: weights + state exceed the device")
        return p
    per_block = kv_block_bytes(cfg, tp, kv_fp8)
    p.blocks = int(blocks if blocks is not None else fit_num_blocks(left, per_block, pool_fraction))
    p.rows["kv pool"] = p.blocks * per_block
    p.rows["prefix state store"] = int(state_bytes) if state_bytes else \
        (int(left * state_fraction * (1 - pool_fraction) * 3) if blocks is None else 0)
    p.notes.append(f"kv pool holds {p.blocks * 16:,} tokens ({p.blocks:,} pages of 16)")
    return p


def _optimizer_state(shapes, optimizer: str) -> Dict[str, int]:
    """fp32 elements of the optimizer state of ``optim.py``: AdamW two moments per parameter;
    Adafactor no first moment and a row + a column vector per matrix (one value per element for
    vectors); ISO a momentum buffer per matrix and Adafactor's state for everything else."""
    first = second = 0
    for shape in shapes:
        n = 1
        for x in shape:
            n *= x
        matrix = len(shape) == 2 and min(shape) >= 2
        if optimizer == "adamw":
            first += n
            second += n
        elif optimizer == "adafactor" or not matrix:
            second += (shape[0] + shape[1]) if matrix else n
        else:                                   # iso, matrix: momentum only
            first += n
    return {"first": first, "second": second}


def train_plan(cfg: ModelConfig, *, mode: str = "lora", rank: int = 16, zero: int = 1, micro_tokens: int = 2048,
               tp: int = 1, optimizer: str = "adamw") -> Dict[str, int]:
    """Bytes per rank of the training-side state.  ``optimizer``: ``adamw`` (two fp32 moments),
    ``adafactor`` (factored second moment, no first moment) or ``iso`` (momentum buffers for the
    matrices, Adafactor for the vectors)."""
    if optimizer not in ("adamw", "adafactor", "iso"):
        raise ValueError(f"unknown optimizer {optimizer!r}")
    n = cfg.n_params()
    rows: Dict[str, int] = {}
    if mode == "lora":
        shapes = []
        for name, (shape, fmt) in weight_specs(cfg).items():
            if fmt in ("nvfp4", "fp8_block") and len(shape) == 2 and name not in ("lm_head",):
                shapes += [(rank, shape[1]), (shape[0], rank)]
        lora = sum(a * b for a, b in shapes)
        rows["adapters (fp32)"] = lora * 4
        rows["grads (fp32)"] = lora * 4
        div = 1
    else:
        shapes = [tuple(shape) for shape, _ in weight_specs(cfg).values()]
        rows["bf16 params"] = n * 2 // zero
        rows["fp32 master"] = n * 4 // zero
        rows["grad shard (fp32)"] = n * 4 // zero
        rows["gathered layer (bf16, x2 buffers)"] = 2 * 2 * (n // max(1, cfg.n_layers))
        div = zero
    st = _optimizer_state(shapes, optimizer)
    if optimizer == "adamw":
        rows["adam moments (fp32 x2)"] = (st["first"] + st["second"]) * 4 // div
    else:
        if st["first"]:
            rows[f"{optimizer} momentum (fp32)"] = st["first"] * 4 // div
        rows[f"{optimizer} second moment (factored, fp32)"] = st["second"] * 4 // div
    rows["tape activations (checkpointed)"] = micro_tokens * cfg.hidden * 2 * (cfg.n_layers + 8)
    return rows


def plan_json(p: Plan, device_bytes: Optional[int] = None) -> Dict[str, object]:
    """The plan's rows as plain data (``serve --dry-run --json``)."""
    out: Dict[str, object] = {"rows": {k: int(v) for k, v in p.rows.items()}, "total_static": int(p.total),
                              "blocks": int(p.blocks), "slots": int(p.slots), "notes": list(p.notes)}
    if device_bytes is not None:
        out["device_bytes"] = int(device_bytes)
        out["free_after"] = int(device_bytes - p.total)
    return out


def memory_table(p: Plan, measured: Optional[Dict[str, int]] = None, peak: Optional[int] = None) -> str:
    wd = max(28, max((len(k) for k in p.rows), default=0) + 1)
    out = [f"{'row':{wd}s} {'derived GiB':>12s} {'measured GiB':>13s}"]
    for k, v in p.rows.items():
        m = (measured or {}).get(k)
        out.append(f"{k:{wd}s} {v / GIB:12.2f} {(m / GIB) if m is not None else float('nan'):13.2f}")
    out.append(f"{'total static':{wd}s} {p.total / GIB:12.2f}")
    if peak is not None:
        out.append(f"{'transient = peak - static':{wd}s} {(peak - p.total) / GIB:12.2f}")
    out += ["# " + n for n in p.notes]
    return "\n".join(out)


def measure(engine) -> Dict[str, int]:
    """Bytes a live engine really holds, under the row names of :func:`plan` (the measured column of
    :func:`memory_table`): weights with their derived layouts, the paged KV pool (and its scales), the
    GDN state slots, the backend's workspace, the prefix store's state snapshots, drafter and indexer."""
    import torch

    def size(t) -> int:
        return t.numel() * t.element_size() if isinstance(t, torch.Tensor) else 0

    def tensors(obj, seen):
        if isinstance(obj, torch.Tensor):
            key = (obj.data_ptr(), obj.numel() * obj.element_size())
            if key not in seen:
                seen.add(key)
                yield obj
        elif isinstance(obj, dict):
            for v in obj.values():
                yield from tensors(v, seen)
        elif isinstance(obj, (list, tuple)):
            for v in obj:
                yield from tensors(v, seen)
        elif hasattr(obj, "__dict__") and type(obj).__module__.startswith("tilerl_b200.formats"):
            yield from tensors(vars(obj), seen)

    out: Dict[str, int] = {}
    seen: set = set()
    out["weights"] = sum(size(t) for t in tensors(getattr(engine.model, "params", {}), seen))
    kv = engine.kv
    out["kv pool"] = sum(size(getattr(kv, a, None)) for a in ("k", "v", "k_scale", "v_scale"))
    st = engine.states
    out["gdn state slots"] = sum(size(getattr(st, a, None)) for a in ("states", "ring", "cur"))
    ws = getattr(engine.ops, "ws", None)
    if ws is not None:
        out["workspace"] = sum(size(t) for t in list(ws.bufs.values()) + list(getattr(ws, "retired", [])))
    if getattr(engine.prefix, "state_bytes", None) is not None:
        out["prefix state store"] = int(engine.prefix.state_bytes)
    d = getattr(engine, "drafter", None)
    if d is not None and hasattr(d, "p"):
        out["drafter parameters"] = sum(size(t) for t in d.p.values())
        out["drafter context (per-request K / V)"] = sum(size(t) for t in tensors([d.ctx, getattr(d, "ctx_kv", {})], set()))
    ix = getattr(getattr(engine, "sparse", None), "indexer", None)
    if ix is not None:
        out["page indexer"] = sum(size(t) for t in ix.parameters())
    return out


def residency(engine) -> Dict[str, int]:
    """Resident bytes of a live engine: ``static`` = the sum of :func:`measure`'s rows, ``peak`` = the
    allocator's high-water mark on the engine's device (on the CPU backend, where nothing keeps one, the
    static sum), ``transient`` = peak - static.  ``serve --record-residency`` appends the three to the bench
    store (reference ``tilerl serve --dry-run --record-residency``, ``src/tilerl/memory.py:542``)."""
    import torch
    static = sum(measure(engine).values())
    dev = torch.device(engine.device)
    peak = int(torch.cuda.max_memory_allocated(dev)) if dev.type == "cuda" else static
    peak = max(peak, static)
    return {"static": int(static), "peak": int(peak), "transient": int(peak - static)}
