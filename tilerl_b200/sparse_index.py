"""Learned page indexer for sparse-KV decode and its warm-up.

Per full-attention layer the indexer holds two small projections: the layer's rotated query
heads ``[hq * D] -> [H, d]`` and a page's mean key ``[hkv * D] -> [H, d]`` (H = 4 heads of
d = 128 by default).  A page's score is ``sum_h relu(q_idx[h] . k_idx[page, h]) / sqrt(d)``
(:func:`tilerl_b200.sparse.learned_index_scores`); the top-k pages by that score replace the
Quest min/max bound when ``SparseKV(indexer=...)`` is given one.

Warm-up (:func:`warmup`): the dense model runs over token batches, a capturing backend records
each attention layer's rotated queries and keys, the *teacher* is the attention mass the dense
softmax puts on every 16-token page (summed over heads), the *student* is
``softmax(page scores)``, and the projections are trained with Adam on ``KL(teacher || student)``.
:func:`topk_recall` measures how much of the teacher's mass the student's top-k pages keep.

The reference's indexer reads hidden-state taps of four source layers
(``src/tilerl/sparse_index.py:153-332``, warm-up ``src/tilerl/train.py:313-713``); this one reads the
attention layer's own q / k, which is what the serving hook already has in hand.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from .ops.ref import KV_BLOCK
from .sparse import learned_index_scores


class LearnedIndexer:
    def __init__(self, cfg, heads: int = 4, dim: int = 128, seed: int = 0, device="cpu", n_q: Optional[int] = None,
                 n_kv: Optional[int] = None):
        self.cfg, self.heads, self.dim = cfg, heads, dim
        nq, nkv, d = n_q or cfg.n_q_heads, n_kv or cfg.n_kv_heads, cfg.head_dim
        g = torch.Generator().manual_seed(seed)
        self.wq: List[torch.Tensor] = []
        self.wk: List[torch.Tensor] = []
        for _ in range(max(1, cfg.n_attn_layers)):
            self.wq.append((torch.randn(nq * d, heads * dim, generator=g) / math.sqrt(nq * d)).to(device))
            self.wk.append((torch.randn(nkv * d, heads * dim, generator=g) / math.sqrt(nkv * d)).to(device))

    def parameters(self) -> List[torch.Tensor]:
        return self.wq + self.wk

    def query(self, layer: int, q: torch.Tensor) -> torch.Tensor:
        """``q [hq, D]`` (or ``[n, hq, D]``) -> ``[H, d]`` (``[n, H, d]``)."""
        flat = q.float().reshape(*q.shape[:-2], -1)
        return (flat @ self.wq[layer]).reshape(*q.shape[:-2], self.heads, self.dim)

    def page_keys(self, layer: int, pages: torch.Tensor) -> torch.Tensor:
        """``pages [P, hkv, 16, D]`` (or pre-pooled ``[P, hkv, D]``) -> ``[P, H, d]``."""
        pooled = pages.float().mean(2) if pages.dim() == 4 else pages.float()
        return (pooled.reshape(pooled.shape[0], -1) @ self.wk[layer]).view(-1, self.heads, self.dim)

    def scores(self, layer: int, q: torch.Tensor, kcache: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
        """Serving hook: scores of the listed pages for one query token."""
        return learned_index_scores(self.query(layer, q), self.page_keys(layer, kcache[table.long()]))

    def state_dict(self) -> Dict[str, torch.Tensor]:
        out = {}
        for i, (a, b) in enumerate(zip(self.wq, self.wk)):
            out[f"indexer.{i}.wq"], out[f"indexer.{i}.wk"] = a.detach().cpu(), b.detach().cpu()
        return out

    def load_state_dict(self, sd: Dict[str, torch.Tensor]) -> None:
        for i in range(len(self.wq)):
            self.wq[i] = sd[f"indexer.{i}.wq"].to(self.wq[i].device)
            self.wk[i] = sd[f"indexer.{i}.wk"].to(self.wk[i].device)


def page_mass(q: torch.Tensor, k: torch.Tensor, qpos: int) -> torch.Tensor:
    """Teacher: attention mass per 16-token page for one query.  ``q [hq, D]``, ``k [T, hkv, D]``
    (keys of positions 0..T-1), causal up to ``qpos``.  Returns ``[ceil((qpos+1)/16)]``, sums to 1."""
    hq, d = q.shape
    hkv = k.shape[1]
    n = qpos + 1
    kk = k[:n].float().repeat_interleave(hq // hkv, 1)                 # [n, hq, D]
    s = torch.einsum("hd,nhd->hn", q.float(), kk) / math.sqrt(d)
    p = torch.softmax(s, -1).mean(0)                                    # [n], over heads
    pages = (n + KV_BLOCK - 1) // KV_BLOCK
    pad = pages * KV_BLOCK - n
    return torch.nn.functional.pad(p, (0, pad)).view(pages, KV_BLOCK).sum(-1)


def _student(ix: LearnedIndexer, layer: int, q: torch.Tensor, k: torch.Tensor, qpos: int) -> torch.Tensor:
    n = qpos + 1
    pages = (n + KV_BLOCK - 1) // KV_BLOCK
    pad = pages * KV_BLOCK - n
    kp = torch.nn.functional.pad(k[:n].float(), (0, 0, 0, 0, 0, pad)).view(pages, KV_BLOCK, *k.shape[1:])
    cnt = torch.full((pages,), float(KV_BLOCK))
    cnt[-1] = KV_BLOCK - pad
    pooled = kp.sum(1) / cnt.to(kp.device)[:, None, None]               # mean over the page's real tokens
    return learned_index_scores(ix.query(layer, q), ix.page_keys(layer, pooled))


def capture_qk(model, ids: torch.Tensor) -> List[Tuple[torch.Tensor, torch.Tensor]]:
    """Dense forward of one sequence ``ids [T]`` on the reference backend; returns, per attention
    layer, the rotated queries ``[T, hq, D]`` and keys ``[T, hkv, D]``."""
    from .batch import Batch
    from .kv import GdnStatePool, PagedKvPool
    from .ops import ref
    from .ops.backend import RefOps
    cfg = model.cfg
    got: List[Tuple[torch.Tensor, torch.Tensor]] = []

    class Capture(RefOps):
        def attention(self, qkv, lp, batch, pool, attn_idx, cfg_, n_q, n_kv):
            q, _, k, _ = ref.attn_prep(qkv, lp["q_norm"], lp["k_norm"], batch.positions, n_q=n_q, n_kv=n_kv,
                                       head_dim=cfg_.head_dim, rotary_dim=cfg_.rotary_dim, theta=cfg_.rope_theta,
                                       eps=cfg_.rms_eps, gated=cfg_.attn_gated)
            got.append((q.detach().float().clone(), k.detach().float().clone()))
            return super().attention(qkv, lp, batch, pool, attn_idx, cfg_, n_q, n_kv)

    t = ids.numel()
    blocks = list(range(1, (t + KV_BLOCK - 1) // KV_BLOCK + 1))
    kv = PagedKvPool(cfg, len(blocks) + 1, dtype=torch.float32, n_kv_heads=model.dims.n_kv)
    st = GdnStatePool(cfg, 2, ring_dtype=torch.float32, n_v_heads=model.dims.gdn_nv or None,
                      n_k_heads=model.dims.gdn_nk or None)
    with torch.no_grad():
        model.forward(Batch.build([dict(tokens=ids.tolist(), start=0, blocks=blocks, slot=1)], "cpu"),
                      Capture(), kv, st, last_only=True)
    return got


def warmup(model, ix: LearnedIndexer, batches: Sequence[torch.Tensor], *, steps: int = 50, lr: float = 3e-3,
           queries_per_seq: int = 8, seed: int = 0) -> List[float]:
    """Train the indexer against the dense page mass.  ``batches``: 1-D token tensors (one
    sequence each).  Returns the KL per step."""
    params = [p.requires_grad_(True) for p in ix.parameters()]
    opt = torch.optim.Adam(params, lr=lr)
    caps = [capture_qk(model, b) for b in batches]
    g = torch.Generator().manual_seed(seed)
    hist = []
    for step in range(steps):
        qk = caps[step % len(caps)]
        t = qk[0][0].shape[0]
        loss = torch.zeros(())
        n = 0
        for layer, (q, k) in enumerate(qk):
            for qpos in torch.randint(2 * KV_BLOCK, t, (queries_per_seq,), generator=g).tolist():
                teacher = page_mass(q[qpos], k, qpos)
                student = torch.log_softmax(_student(ix, layer, q[qpos], k, qpos), -1)
                loss = loss + (teacher * (torch.log(teacher.clamp_min(1e-12)) - student)).sum()
                n += 1
        loss = loss / max(1, n)
        opt.zero_grad()
        loss.backward()
        opt.step()
        hist.append(float(loss.detach()))
    for p in params:
        p.requires_grad_(False)
    return hist


def topk_recall(model, ix: LearnedIndexer, ids: torch.Tensor, top_k: int, n_queries: int = 16, seed: int = 1) -> float:
    """Mean teacher mass kept by the student's top-k pages (1.0 = nothing lost)."""
    qk = capture_qk(model, ids)
    g = torch.Generator().manual_seed(seed)
    t = qk[0][0].shape[0]
    kept = []
    with torch.no_grad():
        for layer, (q, k) in enumerate(qk):
            for qpos in torch.randint(4 * KV_BLOCK, t, (n_queries,), generator=g).tolist():
                teacher = page_mass(q[qpos], k, qpos)
                s = _student(ix, layer, q[qpos], k, qpos)
                idx = torch.topk(s, min(top_k, s.numel())).indices
                kept.append(float(teacher[idx].sum()))
    return sum(kept) / len(kept)


# ---- corpus run: recall before / after over prepared spans ---------------------------------------------------
def load_spans(cdir: str, split: str, max_total: int = 0) -> Dict[str, List[torch.Tensor]]:
    """Spans of a prepared corpus directory: files ``<split>_<label>.jsonl`` whose rows are
    ``{"ctx": length, "ids": [...]}``, grouped by length label.  ``max_total`` > 0 keeps that many spans in
    all, dealt round-robin over the sorted lengths (16 over three lengths -> 6 / 5 / 5), so that a cut run
    is not weighted toward the cheap short spans.  Reference ``src/tilerl/train.py:1306-1331``."""
    import glob
    import itertools
    import json
    import os
    groups: Dict[str, List[torch.Tensor]] = {}
    for path in sorted(glob.glob(os.path.join(cdir, f"{split}_*.jsonl"))):
        with open(path) as f:
            rows = [json.loads(ln) for ln in f if ln.strip()]
        if rows:
            groups[str(rows[0].get("ctx", len(rows[0]["ids"])))] = [torch.tensor(r["ids"], dtype=torch.long) for r in rows]
    if max_total:
        labels = sorted(groups)
        picked = {c: 0 for c in labels}
        for c in itertools.islice(itertools.cycle(labels), max_total):
            if picked[c] < len(groups[c]):
                picked[c] += 1
        groups = {c: groups[c][:picked[c]] for c in labels}
    return groups


def held_recall(model, ix: LearnedIndexer, held: Dict[str, List[torch.Tensor]], k_pages: int, *, q_samples: int = 16,
                q_min_pos: int = 0, seed: int = 1) -> Dict[str, float]:
    """Recall at ``k_pages`` per span length: the share of the dense attention mass that the indexer's top
    pages keep, over ``q_samples`` seeded query positions at or after ``q_min_pos`` in every held span."""
    out: Dict[str, float] = {}
    for label, spans in sorted(held.items()):
        vals = []
        for j, ids in enumerate(spans):
            qk = capture_qk(model, ids)
            t = qk[0][0].shape[0]
            lo = min(max(4 * KV_BLOCK, q_min_pos), t - 1)
            g = torch.Generator().manual_seed(seed + 100003 * j)
            kept = []
            with torch.no_grad():
                for layer, (q, k) in enumerate(qk):
                    for qpos in torch.randint(lo, t, (max(1, q_samples),), generator=g).tolist():
                        teacher = page_mass(q[qpos], k, qpos)
                        s = _student(ix, layer, q[qpos], k, qpos)
                        kept.append(float(teacher[torch.topk(s, min(k_pages, s.numel())).indices].sum()))
            vals.append(sum(kept) / len(kept))
        out[label] = sum(vals) / max(1, len(vals))
    return out


def corpus_run(model, ix: LearnedIndexer, train_groups: Dict[str, List[torch.Tensor]],
               held: Dict[str, List[torch.Tensor]], k_pages: int, *, steps: int, lr: float = 3e-3, q_samples: int = 16,
               q_min_pos: int = 0, seed: int = 0, control: Optional[Dict[str, List[torch.Tensor]]] = None,
               recall_threshold: float = 0.0) -> Dict[str, object]:
    """The indexer's science run: recall at ``k_pages`` per held span length before and after the warm-up,
    the KL curve and the tokens seen; ``control`` (held spans of another corpus) is scored under the same
    trained weights, to show that the recall is not an artefact of one corpus' tokenisation.  ``passed`` is
    the worst after-recall against ``recall_threshold``.  Reference ``src/tilerl/train.py:1295-1360``
    (``_train_indexer_recall``) and ``:622`` (``indexer_warmup_run``)."""
    import itertools
    batches = [b for row in itertools.zip_longest(*train_groups.values()) for b in row if b is not None]
    if not batches:
        raise ValueError("no training spans")
    kw = dict(q_samples=q_samples, q_min_pos=q_min_pos, seed=seed + 1)
    before = held_recall(model, ix, held, k_pages, **kw)
    ctl_before = held_recall(model, ix, control, k_pages, **kw) if control else None
    kl = warmup(model, ix, batches, steps=steps, lr=lr, queries_per_seq=max(1, q_samples // 2), seed=seed)
    after = held_recall(model, ix, held, k_pages, **kw)
    out: Dict[str, object] = {"recall_before": before, "recall_after": after, "kl_curve": kl, "k_pages": k_pages,
                              "tokens_seen": sum(int(batches[s % len(batches)].numel()) for s in range(steps)),
                              "q_samples": q_samples, "q_min_pos": q_min_pos, "di": ix.dim, "heads": ix.heads}
    if control:
        out["control"] = {"recall_before": ctl_before, "recall_after": held_recall(model, ix, control, k_pages, **kw)}
    worst = min(after.values()) if after else 0.0
    out["passed"] = bool(worst >= recall_threshold)
    out["worst_recall_after"] = worst
    return out
