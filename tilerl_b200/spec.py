"""Speculative decoding: drafters and the verify bookkeeping.

The engine verifies a width-W chain ``[last committed token, d1 .. d_{W-1}]`` in ONE trunk
forward (W-wide attention over the paged KV, W recurrent GDN steps with the state after
every step kept in its own plane), samples the trunk's own token at every position with
the same per-position seeds plain decoding would use, accepts the leading run where
sample == draft, and adopts the GDN state plane of the last accepted token.  Greedy and
seeded-sampling outputs are therefore identical with and without a drafter.

Drafters (all expose ``aux_layers`` and ``propose``):

* :class:`BlockDrafter` -- W-wide block drafter: reads three trunk hidden taps, keeps an
  incrementally projected context K/V per request, runs a block of ``[embed(last), mask x
  (W-1)]`` through ``n_layers`` non-causal GQA layers of trunk width and scores every slot
  with the trunk's own lm_head (shared embedding and head).
* :class:`ChainDrafter` -- NextN / MTP style: ``fc([norm(embed(tok)), norm(h_trunk)])`` ->
  one causal layer over its own short cache -> trunk lm_head, unrolled greedily.
* :class:`OracleDrafter` / :class:`ConstantDrafter` -- test and benchmark seams: forced
  full acceptance (drafts = the trunk's greedy continuation, precomputed) and zero
  acceptance.

Parity: reference ``src/tilerl/spec.py`` -- ``verify_lens:133``, ``DraftHead:351``,
``DFlash2Config:903``, ``DFlash2Head:954`` (``step:986``, ``context_kv:1031``,
``block_hidden:1045``, ``paths:1071``); engine ``_verify`` ``src/tilerl/engine.py:2625``.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import torch
import torch.nn.functional as F

from .ops import ref


def verify_lens(drafts: Sequence[int], sampled: Sequence[int]) -> int:
    """Length of the leading run where the trunk's sampled token equals the draft."""
    n = 0
    for d, s in zip(drafts, sampled):
        if d != s:
            break
        n += 1
    return n


def expected_goodput(accept_rate: float, width: int) -> float:
    """Expected committed tokens per verify tick for i.i.d. per-slot acceptance."""
    a = min(max(accept_rate, 0.0), 1.0)
    return sum(a ** k for k in range(width))


@dataclass
class BlockDrafterConfig:
    width: int = 8
    n_layers: int = 2
    n_heads: int = 8
    n_kv_heads: int = 2
    taps: int = 3
    window: int = 64          # context positions the block attends to
    ffn_mult: float = 2.0
    top_k: int = 8            # candidates per slot the selector walk chooses from
    sel_rank: int = 16        # rank of the pairwise (previous token, candidate) selector
    conv_taps: int = 2        # depthwise conv along the block before / after each sub-layer
    conv_group: int = 64      # channels that share one conv coefficient


class BlockDrafter:
    """Random-init or loaded block drafter.  Everything here is small-M work on the
    trunk's width; it runs as torch ops on the engine's device."""

    def __init__(self, model, cfg: Optional[BlockDrafterConfig] = None, seed: int = 0, dtype=torch.float32):
        self.cfg = cfg or BlockDrafterConfig()
        self.model = model
        mc = model.cfg
        h = mc.hidden
        n = mc.n_layers
        self.aux_layers = tuple(sorted({max(0, n // 4 - 1), max(0, n // 2 - 1), n - 1}))[-self.cfg.taps:]
        dev = model.params["embed"].device
        g = torch.Generator(device="cpu").manual_seed(seed)
        c = self.cfg
        self.hd = h // c.n_heads
        ffn = int(h * c.ffn_mult)

        def w(*shape, s=0.02):
            return (torch.randn(*shape, generator=g) * s).to(dev, dtype)
        self.p: Dict[str, torch.Tensor] = {"fc": w(h, len(self.aux_layers) * h), "mask": w(h), "pos": w(c.width, h),
                                           "ctx_norm": torch.ones(h, device=dev, dtype=dtype),
                                           "out_norm": torch.ones(h, device=dev, dtype=dtype)}
        self.groups = max(1, h // c.conv_group)
        self.gsize = h // self.groups
        for i in range(c.n_layers):
            q = f"l{i}."
            self.p[q + "norm1"] = torch.ones(h, device=dev, dtype=dtype)
            self.p[q + "norm2"] = torch.ones(h, device=dev, dtype=dtype)
            self.p[q + "q"] = w(c.n_heads * self.hd, h)
            self.p[q + "kv"] = w(2 * c.n_kv_heads * self.hd, h)
            self.p[q + "o"] = w(h, c.n_heads * self.hd)
            self.p[q + "gate_up"] = w(2 * ffn, h)
            self.p[q + "down"] = w(h, ffn)
            for name in ("attn_conv", "mlp_conv"):
                # [side (before / after the sub-layer), tap, group, channel]: tap 0 starts as the identity
                base = torch.zeros(2, c.conv_taps, self.groups, self.gsize)
                base[:, 0] = 1.0
                self.p[q + name + ".base"] = base.to(dev, dtype)
                self.p[q + name + ".proj"] = w(2 * c.conv_taps * self.groups, h, s=0.002)
        # pairwise selector over the top-k candidates of a slot: score += succ[cand] . (pred[prev] * proj(h));
        # `succ` starts at zero, so an untrained selector is the plain argmax
        self.p["sel.proj"] = w(c.sel_rank, h)
        self.p["sel.pred"] = w(mc.vocab, c.sel_rank)
        self.p["sel.succ"] = torch.zeros(mc.vocab, c.sel_rank, device=dev, dtype=dtype)
        self.ctx: Dict[int, torch.Tensor] = {}         # rid -> context features [n, H] (kept for inspection)
        self.ctx_kv: Dict[int, List[torch.Tensor]] = {}   # rid -> per layer [n, 2, n_kv, hd]: K / V of the context rows

    # ---- engine hooks -------------------------------------------------------------------
    def release(self, rid: int) -> None:
        self.ctx.pop(rid, None)
        self.ctx_kv.pop(rid, None)

    def invalidate(self) -> None:
        self.ctx.clear()
        self.ctx_kv.clear()

    def _embed(self, tok: int) -> torch.Tensor:
        return self.model.params["embed"][tok].to(self.p["fc"].dtype)

    def _head(self, x: torch.Tensor) -> torch.Tensor:
        head = self.model.params["embed" if self.model.cfg.tie_embeddings else "lm_head"]
        w = head if isinstance(head, torch.Tensor) else head.dequant()
        # in the table's own dtype: a float copy of a [vocab, hidden] table per proposal would cost GBs
        return (ref.rmsnorm(x, self.p["out_norm"], 1e-6).to(w.dtype) @ w.t().to(x.device)).float()

    def context_features(self, taps: Dict[int, torch.Tensor], rows: slice) -> torch.Tensor:
        """Project the concatenated trunk taps of the given token rows: [n, H]."""
        cat = torch.cat([taps[l][rows].to(self.p["fc"].dtype) for l in self.aux_layers], dim=-1)
        return ref.rmsnorm(cat @ self.p["fc"].t(), self.p["ctx_norm"], 1e-6).to(self.p["fc"].dtype)

    def _attend(self, q, k, v):
        """Non-causal GQA: q [W, nh, d], k/v [S, nkv, d]."""
        c = self.cfg
        g = c.n_heads // c.n_kv_heads
        qq = q.view(q.shape[0], c.n_kv_heads, g, self.hd)
        s = torch.einsum("whgd,shd->hgws", qq.float(), k.float()) / math.sqrt(self.hd)
        p = torch.softmax(s, -1)
        return torch.einsum("hgws,shd->whgd", p, v.float()).reshape(q.shape[0], -1)

    def context_kv(self, feats: torch.Tensor) -> List[torch.Tensor]:
        """K / V of context rows for every layer: ``[n, H]`` -> per layer ``[n, 2, n_kv, hd]``.  They depend
        on the row's features only (the context carries no position code), so rows are projected once,
        when they enter the context, and appended (parity: the incremental context of spec.py:1005-1017,
        src/tilerl)."""
        c = self.cfg
        return [(feats @ self.p[f"l{i}.kv"].t()).view(feats.shape[0], 2, c.n_kv_heads, self.hd) for i in range(c.n_layers)]

    def _conv(self, x: torch.Tensor, delta: torch.Tensor, base: torch.Tensor) -> torch.Tensor:
        """Grouped depthwise conv along the block's slots with per-slot coefficients: ``x [W, H]``,
        ``delta [W, taps, groups]`` (this slot's offsets), ``base [taps, groups, gsize]``.
        out[j] = sum_tap coef[j, tap] * x[j - tap]; a tap that reaches before slot 0 contributes nothing,
        so nothing of an earlier block leaks in (parity: spec.py:1135-1146, src/tilerl)."""
        w_, taps = x.shape[0], base.shape[0]
        xb = x.float().view(w_, self.groups, self.gsize)
        coef = base.float().unsqueeze(0) + delta.float().unsqueeze(-1)          # [W, taps, groups, gsize]
        out = coef[:, 0] * xb
        for tap in range(1, taps):
            out[tap:] += coef[tap:, tap] * xb[:-tap]
        return out.reshape(w_, -1).to(x.dtype)

    def _conv_in(self, x: torch.Tensor, norm_key: str, conv_key: str):
        """Norm, the conv before the sub-layer, and the offsets of its partner after it (one
        projection yields both sides)."""
        c = self.cfg
        hx = ref.rmsnorm(x, self.p[norm_key], 1e-6).to(x.dtype)
        d = (hx @ self.p[conv_key + ".proj"].t()).view(x.shape[0], 2, c.conv_taps, self.groups)
        return self._conv(hx, d[:, 0], self.p[conv_key + ".base"][0]), d[:, 1]

    def block_hidden(self, last_tok: int, ctx, ctx_kv: Optional[List[torch.Tensor]] = None) -> torch.Tensor:
        """Run the mask-token block over the context; returns [W, H].  ``ctx``: context features
        ``[n, H]``; ``ctx_kv``: their per-layer K / V if the caller keeps them (else projected here)."""
        c = self.cfg
        x = torch.stack([self._embed(last_tok)] + [self.p["mask"]] * (c.width - 1)) + self.p["pos"]
        if ctx_kv is None:
            ctx_kv = self.context_kv(ctx[-c.window:])
        for i in range(c.n_layers):
            q_ = f"l{i}."
            hx, after = self._conv_in(x, q_ + "norm1", q_ + "attn_conv")
            own = (hx @ self.p[q_ + "kv"].t()).view(c.width, 2, c.n_kv_heads, self.hd)
            kv = torch.cat([ctx_kv[i][-c.window:].to(own.dtype), own])       # context rows first, then the block itself
            q = (hx @ self.p[q_ + "q"].t()).view(c.width, c.n_heads, self.hd)
            a = self._attend(q, kv[:, 0], kv[:, 1]).to(x.dtype) @ self.p[q_ + "o"].t()
            x = x + self._conv(a, after, self.p[q_ + "attn_conv.base"][1])
            hx, after = self._conv_in(x, q_ + "norm2", q_ + "mlp_conv")
            gu = hx @ self.p[q_ + "gate_up"].t()
            f = gu.shape[-1] // 2
            m = (F.silu(gu[:, :f]) * gu[:, f:]) @ self.p[q_ + "down"].t()
            x = x + self._conv(m, after, self.p[q_ + "mlp_conv.base"][1])
        return x

    def paths(self, hidden: torch.Tensor, anchor: int) -> List[int]:
        """Top-k candidates per slot from the trunk's head, then one greedy walk: a slot's candidate is
        scored by its logit plus a low-rank pairwise term with the token chosen for the slot before
        (``succ[cand] . (pred[prev] * proj(h))``), so the block is read out sequentially although it
        was computed in parallel (parity: spec.py:1071-1100, src/tilerl)."""
        c = self.cfg
        logits = self._head(hidden)                                            # [slots, vocab]
        unary, cand = torch.topk(logits, min(c.top_k, logits.shape[-1]), dim=-1)
        proj = (hidden.to(self.p["sel.proj"].dtype) @ self.p["sel.proj"].t()).float()   # [slots, r]
        pred, succ = self.p["sel.pred"], self.p["sel.succ"]
        prev, out = torch.as_tensor(int(anchor), device=hidden.device), []
        for j in range(hidden.shape[0]):                                      # on the device: one host sync for the block
            pair = succ[cand[j]].float() @ (pred[prev].float() * proj[j])     # [k]
            prev = cand[j][(unary[j].float() + pair).argmax()]
            out.append(prev)
        return [int(t) for t in torch.stack(out).tolist()] if out else []

    def propose(self, engine, req, taps, tok_off: int, n_run: int, k: int) -> List[int]:
        """Drafts for the next verify tick.  ``taps``: trunk residual-stream taps of this tick's
        tokens; rows ``tok_off .. tok_off + n_valid`` belong to tokens that were really
        committed to the sequence."""
        if taps is None or k <= 0:
            return []
        n_valid = min(n_run, max(1, getattr(req, "n_last_commit", n_run))) if req.state == "decode" and n_run <= \
            engine.spec_width else n_run
        feats = self.context_features(taps, slice(tok_off, tok_off + n_valid))
        old = self.ctx.get(req.rid)
        ctx = (feats if old is None else torch.cat([old, feats]))[-self.cfg.window:]
        self.ctx[req.rid] = ctx
        # only the rows that entered the context this tick are projected to K / V
        new_kv = self.context_kv(feats)
        old_kv = self.ctx_kv.get(req.rid)
        kv = [(n if o is None else torch.cat([o, n]))[-self.cfg.window:] for o, n in zip(old_kv or [None] * len(new_kv), new_kv)]
        self.ctx_kv[req.rid] = kv
        hid = self.block_hidden(req.toks[-1], ctx, kv)
        return self.paths(hid[1:1 + k] if hid.shape[0] > k else hid[-k:], req.toks[-1])[:k]


class ChainDrafter:
    """NextN-style chain drafter sharing the trunk's embedding and lm_head."""

    def __init__(self, model, seed: int = 0, dtype=torch.float32):
        self.model = model
        h = model.cfg.hidden
        self.aux_layers = (model.cfg.n_layers - 1,)
        dev = model.params["embed"].device
        g = torch.Generator(device="cpu").manual_seed(seed)
        self.fc = (torch.randn(h, 2 * h, generator=g) * 0.02).to(dev, dtype)
        self.mix = (torch.randn(h, h, generator=g) * 0.02).to(dev, dtype)
        self.n1 = torch.ones(h, device=dev, dtype=dtype)
        self.n2 = torch.ones(h, device=dev, dtype=dtype)
        self.hidden: Dict[int, torch.Tensor] = {}

    def release(self, rid: int) -> None:
        self.hidden.pop(rid, None)

    def invalidate(self) -> None:
        self.hidden.clear()

    def step(self, tok: int, h_prev: torch.Tensor) -> torch.Tensor:
        e = self.model.params["embed"][tok].to(self.fc.dtype)
        z = torch.cat([ref.rmsnorm(e, self.n1, 1e-6), ref.rmsnorm(h_prev, self.n2, 1e-6)]).to(self.fc.dtype)
        x = z @ self.fc.t()
        return x + F.silu(x @ self.mix.t())

    def propose(self, engine, req, taps, tok_off: int, n_run: int, k: int) -> List[int]:
        if taps is None or k <= 0:
            return []
        n_valid = min(n_run, max(1, getattr(req, "n_last_commit", n_run)))
        h = taps[self.aux_layers[0]][tok_off + n_valid - 1].to(self.fc.dtype)
        head = self.model.params["embed" if self.model.cfg.tie_embeddings else "lm_head"]
        w = (head if isinstance(head, torch.Tensor) else head.dequant()).to(h.device)
        out, tok = [], req.toks[-1]
        for _ in range(k):
            h = self.step(tok, h)
            tok = int((h.to(w.dtype) @ w.t()).float().argmax())
            out.append(tok)
        return out


class OracleDrafter:
    """Forced full acceptance: proposes the continuation recorded for each prompt (the
    trunk's own greedy output).  Used to time the verify tick at acceptance = 1."""
    aux_layers: tuple = ()

    def __init__(self, continuations: Dict[tuple, List[int]]):
        self.cont = continuations

    def propose(self, engine, req, taps, tok_off, n_run, k) -> List[int]:
        c = self.cont.get(tuple(req.prompt))
        if c is None:
            return []
        i = len(req.out)
        return list(c[i:i + k])

    def release(self, rid: int) -> None:
        pass


class ConstantDrafter:
    """Zero acceptance (with overwhelming probability): always proposes the same token."""
    aux_layers: tuple = ()

    def __init__(self, token: int = 0):
        self.token = token

    def propose(self, engine, req, taps, tok_off, n_run, k) -> List[int]:
        return [self.token] * k

    def release(self, rid: int) -> None:
        pass


# ---- drafter checkpoints -------------------------------------------------------------------------
def save_drafter(drafter, path: str) -> None:
    """Writes a block or chain drafter as ``<path>/drafter.safetensors`` plus ``drafter.json``
    (kind, shape-defining config, tap layers)."""
    import dataclasses
    import json
    import os
    from safetensors.torch import save_file
    os.makedirs(path, exist_ok=True)
    if isinstance(drafter, BlockDrafter):
        tensors = {k: v.detach().cpu().contiguous() for k, v in drafter.p.items()}
        meta = {"kind": "block", "config": dataclasses.asdict(drafter.cfg), "aux_layers": list(drafter.aux_layers)}
    elif isinstance(drafter, ChainDrafter):
        tensors = {k: getattr(drafter, k).detach().cpu().contiguous() for k in ("fc", "mix", "n1", "n2")}
        meta = {"kind": "chain", "aux_layers": list(drafter.aux_layers)}
    else:
        raise TypeError(f"{type(drafter).__name__} has no parameters to save")
    meta["hidden"] = int(drafter.model.cfg.hidden)
    save_file(tensors, os.path.join(path, "drafter.safetensors"))
    with open(os.path.join(path, "drafter.json"), "w") as f:
        json.dump(meta, f)


def load_drafter(model, path: str, dtype=torch.float32):
    """The drafter saved by :func:`save_drafter`, bound to ``model`` (its embedding and lm_head) on
    the model's device.  Refuses a drafter trained for another trunk width or tensor shapes that do
    not match the recorded config.
    Parity: reference ``src/tilerl/spec.py:863`` (``load_draft``) and ``:1148`` (``load_dflash2``)."""
    import json
    import os
    from safetensors.torch import load_file
    with open(os.path.join(path, "drafter.json")) as f:
        meta = json.load(f)
    if meta.get("hidden") != int(model.cfg.hidden):
        raise ValueError(f"drafter was built for hidden size {meta.get('hidden')}, the model has {model.cfg.hidden}")
    tensors = load_file(os.path.join(path, "drafter.safetensors"))
    dev = model.params["embed"].device
    if meta["kind"] == "block":
        d = BlockDrafter(model, BlockDrafterConfig(**meta["config"]), dtype=dtype)
        if set(tensors) != set(d.p):
            raise ValueError("drafter checkpoint does not hold the tensors of its recorded config")
        for k, v in tensors.items():
            if tuple(v.shape) != tuple(d.p[k].shape):
                raise ValueError(f"drafter tensor {k} has shape {tuple(v.shape)}, expected {tuple(d.p[k].shape)}")
            d.p[k] = v.to(dev, dtype)
    elif meta["kind"] == "chain":
        d = ChainDrafter(model, dtype=dtype)
        for k in ("fc", "mix", "n1", "n2"):
            if tuple(tensors[k].shape) != tuple(getattr(d, k).shape):
                raise ValueError(f"drafter tensor {k} has the wrong shape")
            setattr(d, k, tensors[k].to(dev, dtype))
    else:
        raise ValueError(f"unknown drafter kind {meta['kind']!r}")
    d.aux_layers = tuple(meta["aux_layers"])
    return d
