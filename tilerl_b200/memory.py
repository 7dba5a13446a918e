"""Memory planner: what fits on a 180 GB B200 (per TP rank) and how the rest is split.

``plan`` prices the served weights (from the format registry), the GDN state slots, the
workspace, and hands ``pool_fraction`` of what remains to the paged KV pool and
``state_fraction`` to the prefix-state store; ``train_plan`` prices adapter / master /
optimizer / gradient / tape bytes for LoRA and ZeRO-3 full-parameter training.
``memory_table`` prints derived vs measured rows with ``transient = peak - sum(static)``.

Parity: reference ``src/tilerl/memory.py:24,48,114,245,411,435,542,680``.
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


def plan(cfg: ModelConfig, *, device_bytes: int = B200_BYTES, tp: int = 1, slots: int = 64, planes: int = 1,
         max_batched_tokens: int = 8192, reserve_bytes: int = 2 * GIB, pool_fraction: float = 2 / 3,
         state_fraction: float = 1 / 4, kv_fp8: bool = False, blocks: Optional[int] = None) -> Plan:
    p = Plan(slots=slots)
    p.rows["weights"] = weight_bytes(cfg, tp)
    p.rows["gdn state slots"] = slots * state_slot_bytes(cfg, tp, planes)
    d = tp_dims(cfg, tp)
    widest = max(d.qkv_rows, d.gdn_in_rows, 2 * d.ffn)
    p.rows["workspace"] = max_batched_tokens * (widest * 2 + cfg.hidden * 8 + d.ffn * 2) + d.vocab_local * 4 * 64
    p.rows["reserve"] = reserve_bytes
    left = device_bytes - p.total
    if left <= 0:
        p.notes.append("model does not fit: weights + state exceed the device")
        return p
    per_block = kv_block_bytes(cfg, tp, kv_fp8)
    p.blocks = int(blocks if blocks is not None else left * pool_fraction // per_block)
    p.rows["kv pool"] = p.blocks * per_block
    p.rows["prefix state store"] = int(left * state_fraction * (1 - pool_fraction) * 3) if blocks is None else 0
    p.notes.append(f"kv pool holds {p.blocks * 16:,} tokens ({p.blocks:,} pages of 16)")
    return p


def train_plan(cfg: ModelConfig, *, mode: str = "lora", rank: int = 16, zero: int = 1, micro_tokens: int = 2048,
               tp: int = 1) -> Dict[str, int]:
    """Bytes per rank of the training-side state."""
    n = cfg.n_params()
    rows: Dict[str, int] = {}
    if mode == "lora":
        lora = 0
        for name, (shape, fmt) in weight_specs(cfg).items():
            if fmt in ("nvfp4", "fp8_block") and len(shape) == 2 and name not in ("lm_head",):
                lora += rank * (shape[0] + shape[1])
        rows["adapters (fp32)"] = lora * 4
        rows["adam moments (fp32 x2)"] = lora * 8
        rows["grads (fp32)"] = lora * 4
    else:
        rows["bf16 params"] = n * 2 // zero
        rows["fp32 master"] = n * 4 // zero
        rows["adam moments (fp32 x2)"] = n * 8 // zero
        rows["grad shard (fp32)"] = n * 4 // zero
        rows["gathered layer (bf16, x2 buffers)"] = 2 * 2 * (n // max(1, cfg.n_layers))
    rows["tape activations (checkpointed)"] = micro_tokens * cfg.hidden * 2 * (cfg.n_layers + 8)
    return rows


def memory_table(p: Plan, measured: Optional[Dict[str, int]] = None, peak: Optional[int] = None) -> str:
    out = [f"{'row':28s} {'derived GiB':>12s} {'measured GiB':>13s}"]
    for k, v in p.rows.items():
        m = (measured or {}).get(k)
        out.append(f"{k:28s} {v / GIB:12.2f} {(m / GIB) if m is not None else float('nan'):13.2f}")
    out.append(f"{'total static':28s} {p.total / GIB:12.2f}")
    if peak is not None:
        out.append(f"{'transient = peak - static':28s} {(peak - p.total) / GIB:12.2f}")
    out += ["# " + n for n in p.notes]
    return "\n".join(out)
