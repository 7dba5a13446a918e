"""Device mesh and tensor-parallel shard tables.

``Mesh(dp, tp, cp)`` places rank ``((dp_i * tp) + tp_i) * cp + cp_i`` and lists the
rank groups of each axis in a fixed order (every rank must create the process
groups in the same order).  ``tp_dims`` gives the per-rank head / row counts and
``shard_param`` slices one full parameter for one TP rank:

* column-parallel (split output rows): ``qkv`` (per head, segments q|k|v),
  GDN ``in`` (segments q|k|v|z|a|b by head), ``gate_up`` (interleaved gate/up
  pairs stay together), ``lm_head`` (vocab rows, zero-padded);
* row-parallel (split the reduction dim): ``o``, ``out``, ``down`` -- their
  partial products are summed across the TP group;
* per-head vectors (``conv``, ``dt_bias``, ``a_log``) follow their heads; norms and
  the embedding table are replicated.

When ``tp > n_kv_heads`` each KV head is replicated on ``tp / n_kv_heads`` ranks.

Parity: reference ``src/tilerl/tensor_parallel.py`` -- split tables ``:33-58``,
``Mesh:60-112``, ``zigzag:115-150``, ``pad_vocab:152``, ``kv_replicas:158``,
``tp_config:238``, ``_check_align:267``, ``shard_params:290``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Tuple

import torch

from ..config import ModelConfig

COLUMN_PARALLEL = ("qkv", "in", "gate_up", "lm_head")
ROW_PARALLEL = ("o", "out", "down")
REPLICATED = ("embed", "final_norm", "norm1", "norm2", "q_norm", "k_norm", "gdn_norm")


@dataclass(frozen=True)
class Mesh:
    dp: int = 1
    tp: int = 1
    cp: int = 1

    @property
    def world(self) -> int:
        return self.dp * self.tp * self.cp

    def rank_of(self, dp_i: int, tp_i: int, cp_i: int = 0) -> int:
        return ((dp_i * self.tp) + tp_i) * self.cp + cp_i

    def coords(self, rank: int) -> Tuple[int, int, int]:
        cp_i = rank % self.cp
        tp_i = (rank // self.cp) % self.tp
        dp_i = rank // (self.cp * self.tp)
        return dp_i, tp_i, cp_i

    def tp_groups(self) -> List[List[int]]:
        return [[self.rank_of(d, t, c) for t in range(self.tp)]
                for d in range(self.dp) for c in range(self.cp)]

    def dp_groups(self) -> List[List[int]]:
        return [[self.rank_of(d, t, c) for d in range(self.dp)]
                for t in range(self.tp) for c in range(self.cp)]

    def cp_groups(self) -> List[List[int]]:
        return [[self.rank_of(d, t, c) for c in range(self.cp)]
                for d in range(self.dp) for t in range(self.tp)]

    def group_of(self, rank: int, axis: str) -> List[int]:
        groups = {"tp": self.tp_groups, "dp": self.dp_groups, "cp": self.cp_groups}[axis]()
        for g in groups:
            if rank in g:
                return g
        raise ValueError(f"rank {rank} outside mesh of {self.world}")


def zigzag_chunks(seq_len: int, cp: int, cp_rank: int) -> List[Tuple[int, int]]:
    """Causal-balanced context-parallel split: the sequence is cut in ``2*cp``
    chunks and rank r owns chunks r and ``2*cp-1-r``.  Returns [(start, end)]."""
    n = 2 * cp
    if seq_len % n:
        raise ValueError(f"seq_len {seq_len} must divide by 2*cp={n}")
    c = seq_len // n
    return [(cp_rank * c, (cp_rank + 1) * c), ((n - 1 - cp_rank) * c, (n - cp_rank) * c)]


def zigzag_positions(seq_len: int, cp: int, cp_rank: int) -> torch.Tensor:
    return torch.cat([torch.arange(a, b) for a, b in zigzag_chunks(seq_len, cp, cp_rank)])


def pad_vocab(vocab: int, tp: int, multiple: int = 64) -> int:
    m = multiple * tp
    return (vocab + m - 1) // m * m


def kv_replicas(n_kv: int, tp: int) -> int:
    return max(1, tp // n_kv)


@dataclass(frozen=True)
class TPDims:
    tp: int
    n_q: int
    n_kv: int
    kv_rep: int
    qkv_rows: int
    gdn_nk: int
    gdn_nv: int
    gdn_conv_dim: int
    gdn_in_rows: int
    ffn: int
    vocab_padded: int
    vocab_local: int


def tp_dims(cfg: ModelConfig, tp: int) -> TPDims:
    if cfg.n_q_heads % tp:
        raise ValueError(f"n_q_heads {cfg.n_q_heads} not divisible by tp {tp}")
    rep = kv_replicas(cfg.n_kv_heads, tp)
    if tp <= cfg.n_kv_heads and cfg.n_kv_heads % tp:
        raise ValueError(f"n_kv_heads {cfg.n_kv_heads} not divisible by tp {tp}")
    if tp > cfg.n_kv_heads and tp % cfg.n_kv_heads:
        raise ValueError(f"tp {tp} must be a multiple of n_kv_heads {cfg.n_kv_heads}")
    n_q = cfg.n_q_heads // tp
    n_kv = max(1, cfg.n_kv_heads // tp)
    d = cfg.head_dim
    nk = nv = 0
    if cfg.n_gdn_layers:
        if cfg.gdn_k_heads % tp or cfg.gdn_v_heads % tp:
            raise ValueError(f"GDN heads ({cfg.gdn_k_heads}/{cfg.gdn_v_heads}) not divisible by tp {tp}")
        nk, nv = cfg.gdn_k_heads // tp, cfg.gdn_v_heads // tp
    if cfg.ffn % tp:
        raise ValueError(f"ffn {cfg.ffn} not divisible by tp {tp}")
    gd = cfg.gdn_head_dim
    conv = 2 * nk * gd + nv * gd
    vp = pad_vocab(cfg.vocab, tp) if tp > 1 else cfg.vocab
    return TPDims(
        tp=tp, n_q=n_q, n_kv=n_kv, kv_rep=rep,
        qkv_rows=n_q * d * (2 if cfg.attn_gated else 1) + 2 * n_kv * d,
        gdn_nk=nk, gdn_nv=nv, gdn_conv_dim=conv, gdn_in_rows=conv + nv * gd + 2 * nv,
        ffn=cfg.ffn // tp, vocab_padded=vp, vocab_local=vp // tp,
    )


def check_alignment(cfg: ModelConfig, tp: int) -> None:
    """Refuse shard shapes the quantised kernels cannot address: NVFP4 needs the
    reduction dim of every shard to be a multiple of 16 (one scale block), the
    block-scaled FP8 format a multiple of 128."""
    d = tp_dims(cfg, tp)
    need = {"nvfp4": 16, "fp8": 128}.get(cfg.quant, 1)
    for name, k in (("o", d.n_q * cfg.head_dim), ("out", d.gdn_nv * cfg.gdn_head_dim), ("down", d.ffn)):
        if k and k % need:
            raise ValueError(f"tp={tp}: reduction dim {k} of '{name}' is not a multiple of {need}")


def shard_dim(name: str) -> int | None:
    leaf = name.split(".")[-1]
    if leaf in COLUMN_PARALLEL or leaf in ("conv", "dt_bias", "a_log"):
        return 0
    if leaf in ROW_PARALLEL:
        return 1
    return None


def is_sharded(name: str) -> bool:
    return shard_dim(name) is not None


def grad_is_sharded(name: str) -> bool:
    """Whether the gradient stored under ``name`` (a parameter name, its ``master.`` copy or a LoRA
    factor) is this rank's shard of a larger tensor -- its squared norm then adds over the TP ranks --
    or a replicated tensor every rank holds whole (counted once).  A LoRA factor follows the split
    of its projection: B with a column-parallel base, A with a row-parallel one."""
    if name.startswith("master."):
        name = name[len("master."):]
    if name.endswith(".lora_a") or name.endswith(".lora_b"):
        base, which = name[:-7], name[-1]
        d = shard_dim(base)
        return (d == 0 and which == "b") or (d == 1 and which == "a")
    return is_sharded(name)


def shard_spec(cfg: ModelConfig, name: str, rank: int, tp: int):
    """How rank ``rank`` cuts parameter ``name``: ``("full",)``, ``("rows", [(a, b), ...], pad_to)``
    (row ranges concatenated, optionally zero-padded to ``pad_to`` source rows first) or
    ``("cols", (a, b))``.  One description serves dense tensors and packed NVFP4 planes."""
    leaf = name.split(".")[-1]
    if tp == 1 or leaf in REPLICATED:
        return ("full",)
    d = tp_dims(cfg, tp)
    hd = cfg.head_dim
    if leaf == "lm_head":
        return ("rows", [(rank * d.vocab_local, (rank + 1) * d.vocab_local)], d.vocab_padded)
    if leaf == "qkv":
        per_q = hd * (2 if cfg.attn_gated else 1)
        q_all = cfg.n_q_heads * per_q
        kv_all = cfg.n_kv_heads * hd
        kv0 = (rank // d.kv_rep) * d.n_kv if tp > cfg.n_kv_heads else rank * d.n_kv
        return ("rows", [(rank * d.n_q * per_q, (rank + 1) * d.n_q * per_q),
                         (q_all + kv0 * hd, q_all + (kv0 + d.n_kv) * hd),
                         (q_all + kv_all + kv0 * hd, q_all + kv_all + (kv0 + d.n_kv) * hd)], None)
    if leaf == "o":
        c = d.n_q * hd
        return ("cols", (rank * c, (rank + 1) * c))
    gd = cfg.gdn_head_dim
    if leaf in ("in", "conv"):
        qd, vd = cfg.gdn_qk_dim, cfg.gdn_v_dim
        lk, lv = d.gdn_nk * gd, d.gdn_nv * gd
        segs = [(rank * lk, (rank + 1) * lk), (qd + rank * lk, qd + (rank + 1) * lk),
                (2 * qd + rank * lv, 2 * qd + (rank + 1) * lv)]
        if leaf == "in":
            base = 2 * qd + vd
            segs.append((base + rank * lv, base + (rank + 1) * lv))
            base += vd
            nv = cfg.gdn_v_heads
            segs.append((base + rank * d.gdn_nv, base + (rank + 1) * d.gdn_nv))
            segs.append((base + nv + rank * d.gdn_nv, base + nv + (rank + 1) * d.gdn_nv))
        return ("rows", segs, None)
    if leaf == "out":
        c = d.gdn_nv * gd
        return ("cols", (rank * c, (rank + 1) * c))
    if leaf in ("dt_bias", "a_log"):
        return ("rows", [(rank * d.gdn_nv, (rank + 1) * d.gdn_nv)], None)
    if leaf == "gate_up":
        return ("rows", [(rank * 2 * d.ffn, (rank + 1) * 2 * d.ffn)], None)
    if leaf == "down":
        return ("cols", (rank * d.ffn, (rank + 1) * d.ffn))
    raise KeyError(f"no shard rule for parameter {name!r}")


def apply_spec(w: torch.Tensor, spec, col_div: int = 1) -> torch.Tensor:
    """Cut ``w`` by ``spec``; ``col_div`` maps logical column indices to stored ones (2 for
    packed nibbles, 16 for per-16 scales)."""
    kind = spec[0]
    if kind == "full":
        return w
    if kind == "cols":
        a, b = spec[1]
        return w[:, a // col_div:b // col_div].contiguous()
    segs, pad_to = spec[1], spec[2]
    if pad_to is not None and pad_to > w.shape[0]:
        w = torch.cat([w, w.new_zeros((pad_to - w.shape[0],) + tuple(w.shape[1:]))])
    return torch.cat([w[a:b] for a, b in segs]).contiguous()


def shard_param(cfg: ModelConfig, name: str, w, rank: int, tp: int):
    """Slice the full parameter ``name`` for TP rank ``rank``.  A quantised weight is cut in
    its packed form (nibbles, block scales; the tensor scale is shared), so every shard holds
    exactly the values of the full quantised tensor."""
    spec = shard_spec(cfg, name, rank, tp)
    if spec[0] == "full":
        return w
    from ..formats import FP8BlockTensor, NVFP4Tensor
    if isinstance(w, NVFP4Tensor):
        sc = apply_spec(w.scale.view(torch.uint8), spec, 16).view(torch.float8_e4m3fn)
        return NVFP4Tensor(apply_spec(w.wq, spec, 2), sc, w.tscale.clone())
    if isinstance(w, FP8BlockTensor):
        raise NotImplementedError("block-scaled FP8 weights are sharded before quantisation")
    return apply_spec(w, spec)


def shard_params(cfg: ModelConfig, params: Dict[str, torch.Tensor], rank: int, tp: int) -> Dict[str, torch.Tensor]:
    check_alignment(cfg, tp)
    return {k: shard_param(cfg, k, v, rank, tp) for k, v in params.items()}
