"""CUDA-graph decode ticks.

One captured graph per batch bucket.  Each bucket owns a *static* input block:
one int32 device buffer holding token ids, positions, slot mapping, KV lengths,
state slots and the block table back to back, mirrored by one pinned host buffer,
so a tick is: fill the pinned block (numpy), one H2D copy, ``cudaGraphLaunch``,
one D2H copy of the argmax row.  Rows that pad a batch up to its bucket point at
the reserved pad slot / pad page, so they can run the full kernels harmlessly.
All graphs share one memory pool.  Because the tensor-parallel reductions are
kernels of ours (not library collectives), a TP tick is captured exactly like a
single-GPU tick.

Parity: reference ``src/tilerl/decode_graph.py`` -- ``GRAPH_BUCKETS:19``,
``DecodeGraph:36`` (``run:112``), ``GraphCapture:348``, ``make_decode_graph:385``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from .batch import Batch
from .ops.ref import KV_BLOCK

GRAPH_BUCKETS = (1, 2, 4, 8, 16, 24, 32, 48, 64, 96, 128)


def bucket_for(n: int, buckets: Sequence[int] = GRAPH_BUCKETS) -> Optional[int]:
    for b in buckets:
        if n <= b:
            return b
    return None


@dataclass
class TickOut:
    logits: Optional[torch.Tensor]
    argmax: Optional[List[int]]


class _Bucket:
    """Static input block + captured graph for one batch size."""

    def __init__(self, b: int, max_blocks: int, device):
        self.b, self.max_blocks = b, max_blocks
        n = 5 * b + b * max_blocks
        self.host = torch.zeros(n, dtype=torch.int32).pin_memory() if device.type == "cuda" \
            else torch.zeros(n, dtype=torch.int32)
        self.np = self.host.numpy()
        self.dev = torch.zeros(n, dtype=torch.int32, device=device)
        v = lambda i: self.dev[i * b:(i + 1) * b]
        ar = torch.arange(b, dtype=torch.int32, device=device)
        self.batch = Batch(
            token_ids=v(0), positions=v(1), seq_ids=ar, slot_mapping=v(2), q_start=ar.clone(),
            q_len=torch.ones(b, dtype=torch.int32, device=device), kv_len=v(3), state_slots=v(4),
            block_table=self.dev[5 * b:].view(b, max_blocks), last_idx=ar.clone(), n_seqs=b, n_tokens=b,
            max_q_len=1, keep_steps=0, host_q_len=[1] * b, host_kv_len=[1] * b,
            keep_rows=[False] * b, keep_flags=torch.zeros(b, dtype=torch.int32, device=device))
        self.graph = None
        self.out_tok: Optional[torch.Tensor] = None
        self.out_logits: Optional[torch.Tensor] = None
        self.tok_host = torch.zeros(b, dtype=torch.int32).pin_memory() if device.type == "cuda" \
            else torch.zeros(b, dtype=torch.int32)
        self.hist_cap = 256
        self.hist = torch.zeros(b, self.hist_cap, dtype=torch.int32, device=device)
        self.hist_n = torch.zeros(1, dtype=torch.int32, device=device)
        self.kernels = 0

    def fill(self, seqs: Sequence[dict]) -> None:
        b, mb, a = self.b, self.max_blocks, self.np
        a[:] = 0  # pad rows: token 0, position 0, slot row 0 of page 0, state slot 0
        for r, s in enumerate(seqs):
            pos = int(s["start"])
            blocks = s["blocks"]
            a[r] = s["tokens"][0]
            a[b + r] = pos
            a[2 * b + r] = blocks[pos // KV_BLOCK] * KV_BLOCK + pos % KV_BLOCK
            a[3 * b + r] = pos + 1
            a[4 * b + r] = s["slot"]
            a[5 * b + r * mb: 5 * b + r * mb + len(blocks)] = blocks
        self.h2d_bytes = a.nbytes


class DecodeGraphRunner:
    def __init__(self, model, ops, kv_pool, state_pool, *, max_ctx: int, buckets=GRAPH_BUCKETS,
                 enabled: bool = True):
        self.model, self.ops, self.kv, self.states = model, ops, kv_pool, state_pool
        self.device = kv_pool.k.device
        self.max_blocks = (max_ctx + KV_BLOCK - 1) // KV_BLOCK
        self.buckets = tuple(buckets)
        self.enabled = enabled and self.device.type == "cuda"
        self._b: Dict[int, _Bucket] = {}
        self._pool = None
        self.h2d_bytes = 0
        self.d2h_bytes = 0
        self.replays = 0

    def _splits_for(self, b: int) -> int:
        sms = getattr(self.ops, "sms", 148)
        return max(1, min(64, sms // max(1, b * self.model.dims.n_kv)))

    def _forward(self, bk: _Bucket):
        self.ops.attn_splits = self._splits_for(bk.b)
        logits = self.model.forward(bk.batch, self.ops, self.kv, self.states, last_only=True)
        tok = self.ops.argmax(logits)
        self.ops.attn_splits = 0
        if self.device.type == "cuda":
            from .ops import native as N
            b = bk.batch
            N.check(self.ops.lib.trl_decode_advance(
                tok.data_ptr(), b.token_ids.data_ptr(), b.positions.data_ptr(), b.slot_mapping.data_ptr(),
                b.kv_len.data_ptr(), b.block_table.data_ptr(), bk.b, bk.max_blocks, bk.hist.data_ptr(),
                bk.hist_cap, bk.hist_n.data_ptr(), N.stream()), "decode_advance")
            N.count()
        return logits, tok

    def _capture(self, b: int) -> _Bucket:
        bk = _Bucket(b, self.max_blocks, self.device)
        bk.fill([])
        bk.dev.copy_(bk.host)
        if self.device.type != "cuda":
            self._b[b] = bk
            return bk
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(2):
                self._forward(bk)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        if self._pool is None:
            self._pool = torch.cuda.graph_pool_handle()
        from .ops import native as N
        before = N.launch_count
        with torch.cuda.graph(g, pool=self._pool):
            logits, tok = self._forward(bk)
        bk.kernels = N.launch_count - before
        bk.graph, bk.out_logits, bk.out_tok = g, logits, tok
        self._b[b] = bk
        return bk

    def precapture(self, batches: Sequence[int] = (1,)) -> None:
        for n in batches:
            b = bucket_for(n, self.buckets)
            if b is not None and b not in self._b:
                self._capture(b)

    def run(self, seqs: Sequence[dict]) -> Optional[TickOut]:
        if not self.enabled:
            return None
        b = bucket_for(len(seqs), self.buckets)
        if b is None or any(len(s["blocks"]) > self.max_blocks or len(s["tokens"]) != 1 for s in seqs):
            return None
        bk = self._b.get(b) or self._capture(b)
        bk.fill(seqs)
        bk.dev.copy_(bk.host, non_blocking=True)
        bk.graph.replay()
        bk.tok_host.copy_(bk.out_tok, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        self.replays += 1
        self.h2d_bytes += bk.h2d_bytes
        self.d2h_bytes += bk.tok_host.numel() * 4
        n = len(seqs)
        return TickOut(bk.out_logits[:n], bk.tok_host[:n].tolist())

    def run_device_loop(self, seqs: Sequence[dict], ticks: int) -> List[List[int]]:
        """Greedy-decode ``ticks`` tokens per row with no host round trip between
        ticks: the captured tick ends with a device-side advance kernel, so the
        graph is simply replayed back to back.  Returns the generated tokens."""
        b = bucket_for(len(seqs), self.buckets)
        bk = self._b.get(b) or self._capture(b)
        assert ticks <= bk.hist_cap
        bk.fill(seqs)
        bk.dev.copy_(bk.host, non_blocking=True)
        bk.hist_n.zero_()
        for _ in range(ticks):
            bk.graph.replay()
        self.replays += ticks
        out = bk.hist[:len(seqs), :ticks].cpu()
        return out.tolist()

    def bucket(self, n: int) -> "_Bucket":
        b = bucket_for(n, self.buckets)
        return self._b.get(b) or self._capture(b)


@dataclass
class VerifyOut:
    logits: torch.Tensor                 # [rows, vocab] in the engine's (compact) row order
    argmax: List[int]
    taps: Optional[Dict[int, torch.Tensor]]
    # drafts each sequence's trunk reproduced under greedy acceptance, counted on the device, which has
    # also selected the matching GDN state plane; None when the backend has no such kernel
    accept: Optional[List[int]] = None


class _VBucket:
    """Static input block + captured graph of a width-``w`` verify tick for ``b`` sequences.
    Row layout: sequence ``r`` owns token rows ``r*w .. r*w + w - 1``; a chain shorter than ``w``
    leaves its tail rows as pad tokens (page 0, position 0) outside every ``q_len``."""

    def __init__(self, b: int, w: int, max_blocks: int, device):
        self.b, self.w, self.max_blocks = b, w, max_blocks
        t = b * w
        n = 3 * t + 4 * b + b * max_blocks
        self.host = torch.zeros(n, dtype=torch.int32).pin_memory() if device.type == "cuda" \
            else torch.zeros(n, dtype=torch.int32)
        self.np = self.host.numpy()
        self.dev = torch.zeros(n, dtype=torch.int32, device=device)
        tv = lambda i: self.dev[i * t:(i + 1) * t]
        bv = lambda i: self.dev[3 * t + i * b:3 * t + (i + 1) * b]
        ar = torch.arange(b, dtype=torch.int32, device=device)
        self.batch = Batch(
            token_ids=tv(0), positions=tv(1), seq_ids=ar.repeat_interleave(w).contiguous(), slot_mapping=tv(2),
            q_start=(ar * w).contiguous(), q_len=bv(0), kv_len=bv(1), state_slots=bv(2),
            block_table=self.dev[3 * t + 4 * b:].view(b, max_blocks), last_idx=(ar * w + w - 1).contiguous(),
            n_seqs=b, n_tokens=t, max_q_len=w, keep_steps=w, host_q_len=[w] * b, host_kv_len=[1] * b,
            keep_rows=[True] * b, keep_flags=bv(3))
        self.graph = None
        self.out_tok = self.out_logits = self.out_pack = None
        self.out_taps: Optional[Dict[int, torch.Tensor]] = None
        self.tok_host = torch.zeros(t + b, dtype=torch.int32).pin_memory() if device.type == "cuda" \
            else torch.zeros(t + b, dtype=torch.int32)      # [argmax of every row ; accept count of every sequence]
        self.kernels = 0
        self.h2d_bytes = 0

    def fill(self, seqs: Sequence[dict]) -> List[int]:
        """Returns the row index (in the padded layout) of every real token, in engine order."""
        b, w, mb, a = self.b, self.w, self.max_blocks, self.np
        t = b * w
        a[:] = 0
        rows: List[int] = []
        for r, s in enumerate(seqs):
            toks, start, blocks = s["tokens"], int(s["start"]), s["blocks"]
            for k, tok in enumerate(toks):
                pos = start + k
                a[r * w + k] = tok
                a[t + r * w + k] = pos
                a[2 * t + r * w + k] = blocks[pos // KV_BLOCK] * KV_BLOCK + pos % KV_BLOCK
                rows.append(r * w + k)
            a[3 * t + r] = len(toks)
            a[3 * t + b + r] = start + len(toks)
            a[3 * t + 2 * b + r] = s["slot"]
            a[3 * t + 3 * b + r] = 1
            o = 3 * t + 4 * b + r * mb
            a[o:o + len(blocks)] = blocks
        self.h2d_bytes = a.nbytes
        return rows


class VerifyGraphRunner:
    """CUDA-graph capture of speculative verify ticks (width ``w`` chains): the same forward the
    eager path runs -- W-wide attention, GDN with a state plane per step, logits and argmax of
    every row, the drafter's hidden taps -- replayed from one graph per batch bucket."""

    def __init__(self, model, ops, kv_pool, state_pool, *, max_ctx: int, width: int, aux_layers: Sequence[int] = (),
                 buckets=(1, 2, 4, 8, 16)):
        self.model, self.ops, self.kv, self.states = model, ops, kv_pool, state_pool
        self.device = kv_pool.k.device
        self.max_blocks = (max_ctx + KV_BLOCK - 1) // KV_BLOCK
        self.w, self.aux = int(width), tuple(aux_layers)
        self.buckets = tuple(buckets)
        self.enabled = self.device.type == "cuda"
        self._b: Dict[int, _VBucket] = {}
        self._pool = None
        self.h2d_bytes = self.d2h_bytes = self.replays = 0

    def _forward(self, bk: _VBucket):
        sms = getattr(self.ops, "sms", 148)
        self.ops.attn_splits = max(1, min(32, sms // max(1, bk.b * bk.w * self.model.dims.n_kv)))
        res = self.model.forward(bk.batch, self.ops, self.kv, self.states, last_only=False, aux_layers=self.aux)
        self.ops.attn_splits = 0
        logits, taps = (res[0], res[2]) if self.aux else (res, None)
        tok = self.ops.argmax(logits)
        pack = None
        if hasattr(self.ops, "spec_accept") and getattr(self.states, "cur", None) is not None:
            # accept length per sequence and the state-plane selection, inside the graph
            pack = self.ops.ws.get(f"spec_pack_{bk.b}", (bk.b * bk.w + bk.b,), torch.int32)
            self.ops.spec_accept(tok, bk.batch, self.states.cur, pack)
        return logits, tok, taps, pack

    def _capture(self, b: int) -> _VBucket:
        bk = _VBucket(b, self.w, self.max_blocks, self.device)
        bk.fill([])
        bk.dev.copy_(bk.host)
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(2):
                self._forward(bk)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        if self._pool is None:
            self._pool = torch.cuda.graph_pool_handle()
        from .ops import native as N
        before = N.launch_count
        with torch.cuda.graph(g, pool=self._pool):
            logits, tok, taps, pack = self._forward(bk)
        bk.kernels = N.launch_count - before
        bk.graph, bk.out_logits, bk.out_tok, bk.out_taps, bk.out_pack = g, logits, tok, taps, pack
        self._b[b] = bk
        return bk

    def run(self, seqs: Sequence[dict], need_logits: bool) -> Optional[VerifyOut]:
        if not self.enabled:
            return None
        b = bucket_for(len(seqs), self.buckets)
        if b is None or any(len(s["blocks"]) > self.max_blocks or not 1 <= len(s["tokens"]) <= self.w for s in seqs):
            return None
        bk = self._b.get(b) or self._capture(b)
        rows = bk.fill(seqs)
        bk.dev.copy_(bk.host, non_blocking=True)
        bk.graph.replay()
        t = bk.b * bk.w
        if bk.out_pack is not None:
            bk.tok_host.copy_(bk.out_pack, non_blocking=True)
        else:
            bk.tok_host[:t].copy_(bk.out_tok, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        self.replays += 1
        self.h2d_bytes += bk.h2d_bytes
        self.d2h_bytes += (bk.tok_host.numel() if bk.out_pack is not None else t) * 4
        th = bk.tok_host.tolist()
        accept = th[t:t + len(seqs)] if bk.out_pack is not None else None
        idx = torch.tensor(rows, dtype=torch.long, device=self.device) if (need_logits or bk.out_taps) else None
        taps = {l: v[idx] for l, v in bk.out_taps.items()} if bk.out_taps else None
        logits = bk.out_logits[idx] if need_logits else bk.out_logits
        return VerifyOut(logits, [th[r] for r in rows], taps, accept)
