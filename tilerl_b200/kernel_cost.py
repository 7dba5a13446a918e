"""Declarative cost model: bytes and FLOPs of every kernel of a decode tick and of a
prefill, and the roofline bound they imply.

Every row is ``(name, count, bytes, flops, comm_bytes)`` for ONE rank; ``bound_seconds``
is ``max(bytes / hbm_bw, flops / peak, comm_bytes / nvlink_bw)`` summed over rows, which is
the floor a tick can reach if every kernel sat on its roofline.  The same table prices a
model without a GPU (``cli bench --kernels``) and normalises measured kernel times.

Parity: reference ``src/tilerl/kernel_cost.py`` -- ``TickShape:28``, ``_gemv:45``,
``_paged_attention_decode:92``, ``_gdn_decode_fused:107``, ``prefill_rows:239``,
``tick_rows:292``, ``sparse_indexer_rows:357``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional

from .config import ATTN, ModelConfig
from .formats import FORMATS, nbytes
from .parallel.mesh import tp_dims


@dataclass(frozen=True)
class TickShape:
    batch: int = 1
    ctx: int = 512          # KV length attended per sequence
    width: int = 1          # tokens per sequence in the tick (speculative verify: W)
    tp: int = 1
    sparse_pages: int = 0   # >0: attention reads this many pages instead of ctx/16


@dataclass
class Row:
    name: str
    count: int
    bytes: float
    flops: float
    comm_bytes: float = 0.0

    def bound(self, hbm: float, peak: float, link: float) -> float:
        return self.count * max(self.bytes / hbm, self.flops / peak, self.comm_bytes / link if link else 0.0)


def _lin_format(cfg: ModelConfig) -> str:
    return {"nvfp4": "nvfp4", "fp8": "fp8_block", "bf16": "bf16"}[cfg.quant]


def _linear(name: str, count: int, m: int, n: int, k: int, fmt: str, comm: float = 0.0) -> Row:
    w = nbytes(fmt, (n, k))
    act = m * k * 2 + m * n * 2
    return Row(name, count, w + act, 2.0 * m * n * k, comm)


def tick_rows(cfg: ModelConfig, s: TickShape) -> List[Row]:
    """One decode (or verify) tick on one TP rank."""
    d = tp_dims(cfg, s.tp)
    m = s.batch * s.width
    h = cfg.hidden
    fmt = _lin_format(cfg)
    na, ng = cfg.n_attn_layers, cfg.n_gdn_layers
    ar = (s.tp - 1) * m * h * 4.0 if s.tp > 1 else 0.0      # one-shot all-reduce: fp32 partial to every peer
    rows = [Row("embedding", 1, m * h * 2 * 2, 0)]
    if na:
        hd = cfg.head_dim
        rows.append(_linear("attn.qkv (norm fused)", na, m, d.qkv_rows, h, fmt))
        kv_tokens = (s.sparse_pages * 16 if s.sparse_pages else s.ctx)
        kv_bytes = s.batch * kv_tokens * d.n_kv * hd * 2 * 2
        rows.append(Row("attn.prep + kv write", na, m * d.qkv_rows * 2 + m * d.n_kv * hd * 4, 0))
        rows.append(Row("attn.paged (split + combine)", na, kv_bytes + m * d.n_q * hd * 4,
                        4.0 * m * d.n_q * hd * kv_tokens))
        rows.append(_linear("attn.o (+residual, all-reduce)", na, m, h, d.n_q * hd, fmt, ar))
    if ng:
        gd = cfg.gdn_head_dim
        state = s.batch * d.gdn_nv * gd * gd * 4
        rows.append(_linear("gdn.in (norm fused)", ng, m, d.gdn_in_rows, h, fmt))
        rows.append(Row("gdn.step (state r/w)", ng, state * (1 + s.width) + m * d.gdn_in_rows * 2,
                        6.0 * m * d.gdn_nv * gd * gd))
        rows.append(_linear("gdn.out (+residual, all-reduce)", ng, m, h, d.gdn_nv * gd, fmt, ar))
    rows.append(_linear("mlp.gate_up (norm + swiglu fused)", cfg.n_layers, m, 2 * d.ffn, h, fmt))
    rows.append(_linear("mlp.down (+residual, all-reduce)", cfg.n_layers, m, h, d.ffn, fmt, ar))
    head_fmt = "nvfp4" if cfg.lm_head_quant == "nvfp4" else "bf16"
    rows.append(_linear("lm_head", 1, s.batch, d.vocab_local, h, head_fmt))
    rows.append(Row("argmax", 1, s.batch * d.vocab_local * 4, 0, (s.tp - 1) * s.batch * 8.0 if s.tp > 1 else 0))
    return rows


def prefill_rows(cfg: ModelConfig, tokens: int, tp: int = 1, terms: int = 2) -> List[Row]:
    """One prefill of ``tokens`` tokens (one sequence) on one TP rank; ``terms`` NVFP4
    activation terms per token multiply the tensor-core work."""
    d = tp_dims(cfg, tp)
    h, m = cfg.hidden, tokens
    fmt = _lin_format(cfg)
    na, ng = cfg.n_attn_layers, cfg.n_gdn_layers
    rs = 2.0 * (tp - 1) / tp * m * h * 2 if tp > 1 else 0.0     # reduce-scatter + all-gather of bf16 rows

    def lin(name, count, n, k, comm=0.0):
        r = _linear(name, count, m, n, k, fmt, comm)
        r.flops *= terms
        return r
    rows = [Row("embedding", 1, m * h * 4, 0)]
    if na:
        hd = cfg.head_dim
        rows += [lin("attn.qkv", na, d.qkv_rows, h),
                 Row("attn.causal", na, m * (d.n_q + 2 * d.n_kv) * hd * 2 * 2, 2.0 * m * m * d.n_q * hd),
                 lin("attn.o", na, h, d.n_q * hd, rs)]
    if ng:
        gd = cfg.gdn_head_dim
        rows += [lin("gdn.in", ng, d.gdn_in_rows, h),
                 Row("gdn.scan", ng, m * d.gdn_in_rows * 2 * 2 + d.gdn_nv * gd * gd * 8, 6.0 * m * d.gdn_nv * gd * gd),
                 lin("gdn.out", ng, h, d.gdn_nv * gd, rs)]
    rows += [lin("mlp.gate_up", cfg.n_layers, 2 * d.ffn, h), lin("mlp.down", cfg.n_layers, h, d.ffn, rs)]
    rows.append(_linear("lm_head (last token)", 1, 1, d.vocab_local, h, "bf16"))
    return rows


def sparse_indexer_rows(cfg: ModelConfig, ctx: int, batch: int = 1, tp: int = 1) -> List[Row]:
    d = tp_dims(cfg, tp)
    pages = ctx // 16
    b = batch * pages * d.n_kv * 2 * cfg.head_dim * 2
    return [Row("quest bounds + scores + top-k", cfg.n_attn_layers, b, 4.0 * batch * pages * d.n_q * cfg.head_dim)]


def bound_seconds(rows: List[Row], hbm_gbs: float, peak_tflops: float, nvlink_gbs: float = 770.0) -> float:
    return sum(r.bound(hbm_gbs * 1e9, peak_tflops * 1e12, nvlink_gbs * 1e9) for r in rows)


def tick_bytes(rows: List[Row]) -> float:
    return sum(r.count * r.bytes for r in rows)


def table(rows: List[Row], hbm_gbs: float, peak_tflops: float, nvlink_gbs: float = 770.0,
          measured_us: Optional[Dict[str, float]] = None) -> str:
    out = [f"{'kernel':40s} {'n':>4s} {'MB':>10s} {'GFLOP':>10s} {'bound us':>10s} {'meas us':>10s} {'frac':>6s}"]
    for r in rows:
        b = r.bound(hbm_gbs * 1e9, peak_tflops * 1e12, nvlink_gbs * 1e9) * 1e6
        meas = (measured_us or {}).get(r.name)
        out.append(f"{r.name:40s} {r.count:4d} {r.count * r.bytes / 1e6:10.2f} {r.count * r.flops / 1e9:10.2f} "
                   f"{b:10.1f} {meas if meas is not None else float('nan'):10.1f} "
                   f"{(b / meas) if meas else float('nan'):6.2f}")
    out.append(f"{'total':40s} {'':4s} {tick_bytes(rows) / 1e6:10.2f} {'':10s} "
               f"{bound_seconds(rows, hbm_gbs, peak_tflops, nvlink_gbs) * 1e6:10.1f}")
    return "\n".join(out)
