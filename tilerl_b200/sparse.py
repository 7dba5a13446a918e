"""Top-k sparse KV attention for long-context decode (Quest-style page index).

For every full 16-token page and KV head the index keeps the element-wise min and max
of the keys.  At decode, the upper bound ``sum_d max(q_d * kmin_d, q_d * kmax_d)`` (summed
over the query heads) scores every earlier page; the ``top_k`` best pages plus a trailing
``window`` of recent pages are kept, in sequence order, and attention runs on a *packed*
block table ``[selected pages ; trailing pages]`` with the packed length as the causal
bound -- the same paged-attention kernel, reading ~``(top_k + window) * 16`` keys instead of
the whole context.  The selection is refreshed every ``refresh_ticks`` ticks and reused in
between (new tokens always land in the trailing window).  Selection runs as device tensor
ops (bounds, scores, top-k, sort) without a host round trip; a learned indexer can replace
the Quest scores through ``score_fn``.

Sequences shorter than ``min_tokens`` (or any tick that is not decode-only) use dense
attention, so a server can leave this on and pay nothing for short chats.

Parity: reference ``src/tilerl/sparse_engine.py`` -- ``quest_scores:107``,
``select_members:152``, ``order_members:181``, ``SparseTracker:222``,
``SparseForward:513`` (``attention_args:879``); ``src/tilerl/sparse_index.py:153-332``
(learned indexer maths); page bounds ``tilerl_kernels/reference.py:421-502``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, List, Optional, Tuple

import torch

from .ops.ref import KV_BLOCK


@dataclass
class SparseConfig:
    top_k: int = 128
    window: int = 8
    refresh_ticks: int = 8
    min_tokens: int = 4096


def quest_scores(q: torch.Tensor, bounds: torch.Tensor) -> torch.Tensor:
    """``q [hq, D]``, ``bounds [P, hkv, 2, D]`` -> upper-bound score per page ``[P]``."""
    hkv = bounds.shape[1]
    qg = q.float().view(hkv, -1, q.shape[-1])                       # [hkv, g, D]
    lo = qg[None] * bounds[:, :, None, 0, :].float()
    hi = qg[None] * bounds[:, :, None, 1, :].float()
    return torch.maximum(lo, hi).sum(-1).sum((1, 2))


def learned_index_scores(q_idx: torch.Tensor, k_idx: torch.Tensor) -> torch.Tensor:
    """Learned indexer: ``sum_h relu(q_idx[h] . k_idx[p, h]) / sqrt(d)`` -> ``[P]``.
    ``q_idx [H, d]``, ``k_idx [P, H, d]`` (page-pooled index keys)."""
    d = q_idx.shape[-1]
    return torch.relu(torch.einsum("hd,phd->ph", q_idx.float(), k_idx.float())).sum(-1) / d ** 0.5


def select_pages(scores: torch.Tensor, n_pages: int, top_k: int, window: int) -> torch.Tensor:
    """Indices (ascending) of the kept pages: top-k of the early pages united with the
    trailing window.  Device tensor in, device tensor out."""
    n_win = min(window, n_pages)
    early = n_pages - n_win
    tail = torch.arange(early, n_pages, device=scores.device)
    if early <= 0 or top_k <= 0:
        return tail
    k = min(top_k, early)
    top = torch.topk(scores[:early], k).indices
    return torch.cat([torch.sort(top).values, tail])


class _View:
    """Per-tick sparse view handed to the ops backend through ``batch.sparse``."""

    def __init__(self, mgr: "SparseKV", batch, rids: List[int], use: List[bool]):
        self.mgr, self.batch, self.rids, self.use = mgr, batch, rids, use

    def active(self, attn_idx: int) -> bool:
        return any(self.use)

    def packed(self, attn_idx: int, q: torch.Tensor, kcache: torch.Tensor, ops=None) -> Tuple[torch.Tensor, torch.Tensor]:
        """Packed block table ``[B, P]`` and the causal bound ``packed_len - 1`` per token.  ``ops``: a
        backend with ``quest_select`` scores and selects on the device (two kernels per refresh)."""
        b = self.batch
        rows, lens = [], []
        for r, rid in enumerate(self.rids):
            kv_len = b.host_kv_len[r]
            n_pages = (kv_len + KV_BLOCK - 1) // KV_BLOCK
            table = b.block_table[r, :n_pages]
            if not self.use[r]:
                rows.append(table)
                lens.append(kv_len)
                continue
            sel = self.mgr.selection(rid, attn_idx, q[r], table, kcache, n_pages, ops=ops)   # decode-only: token r
            rows.append(table[sel])
            tail_tokens = kv_len - (n_pages - 1) * KV_BLOCK      # tokens in the last (own) page
            lens.append((sel.numel() - 1) * KV_BLOCK + tail_tokens)
        width = max(int(t.numel()) for t in rows)
        out = torch.zeros(len(rows), width, dtype=torch.int32, device=b.block_table.device)
        for i, t in enumerate(rows):
            out[i, :t.numel()] = t
        pos = torch.tensor([l - 1 for l in lens], dtype=torch.int32, device=b.positions.device)
        return out, pos


class SparseKV:
    def __init__(self, cfg, config: Optional[SparseConfig] = None, score_fn: Optional[Callable] = None,
                 indexer=None):
        self.cfg = cfg
        self.c = config or SparseConfig()
        self.score_fn = score_fn or quest_scores
        self.indexer = indexer            # a sparse_index.LearnedIndexer replaces the Quest bound
        self._sel: Dict[Tuple[int, int], torch.Tensor] = {}     # (rid, layer) -> kept early pages
        self._age: Dict[Tuple[int, int], int] = {}
        self._early: Dict[Tuple[int, int], int] = {}
        self.stats = dict(sparse_ticks=0, dense_ticks=0, refreshes=0, device_selects=0)

    # engine hooks ---------------------------------------------------------------------------
    def for_batch(self, batch, rids: List[int]):
        if batch.max_q_len != 1:
            self.stats["dense_ticks"] += 1
            return None
        use = [kv >= self.c.min_tokens for kv in batch.host_kv_len]
        if not any(use):
            self.stats["dense_ticks"] += 1
            return None
        self.stats["sparse_ticks"] += 1
        return _View(self, batch, rids, use)

    def release(self, rid: int) -> None:
        for k in [k for k in self._sel if k[0] == rid]:
            self._sel.pop(k, None)
            self._age.pop(k, None)
            self._early.pop(k, None)

    # selection --------------------------------------------------------------------------------
    def page_bounds(self, kcache: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
        """``[P, hkv, 2, D]`` min / max over each listed page's 16 tokens."""
        pages = kcache[table.long()].float()                     # [P, hkv, 16, D]
        return torch.stack([pages.amin(2), pages.amax(2)], dim=2)

    def selection(self, rid: int, layer: int, q: torch.Tensor, table: torch.Tensor, kcache: torch.Tensor,
                  n_pages: int, ops=None) -> torch.Tensor:
        """Kept page indices (ascending, ending with the sequence's trailing window)."""
        key = (rid, layer)
        n_win = min(self.c.window, n_pages)
        early = n_pages - n_win
        age = self._age.get(key, self.c.refresh_ticks)
        cached = self._sel.get(key)
        if cached is None or age >= self.c.refresh_ticks:
            if early > 0 and self.c.top_k > 0:
                k = min(self.c.top_k, early)
                cached = None
                if self.indexer is None and self.score_fn is quest_scores and hasattr(ops, "quest_select"):
                    cached = ops.quest_select(q, kcache, table[:early], k)      # device: score + select, two kernels
                    if cached is not None:
                        self.stats["device_selects"] += 1
                if cached is None and self.indexer is not None and hasattr(ops, "index_select"):
                    cached = ops.index_select(self.indexer, layer, q, kcache, table[:early], k)
                    if cached is not None:
                        self.stats["device_selects"] += 1
                if cached is None:
                    if self.indexer is not None:
                        scores = self.indexer.scores(layer, q, kcache, table[:early])
                    else:
                        scores = self.score_fn(q, self.page_bounds(kcache, table[:early]))
                    cached = torch.sort(torch.topk(scores, k).indices).values
            else:
                cached = torch.zeros(0, dtype=torch.long, device=table.device)
            self._sel[key] = cached
            self._early[key] = early
            self._age[key] = 0
            self.stats["refreshes"] += 1
        self._age[key] = self._age.get(key, 0) + 1
        # pages that slid out of the window since the last refresh stay attended until the next one
        tail = torch.arange(min(self._early.get(key, early), early), n_pages, device=table.device)
        return torch.cat([cached.to(table.device), tail])
