"""Per-forward batch descriptor (flat-token layout).

A tick's tokens from all scheduled sequences are concatenated into ``[T]``.
Decode ticks have one token per sequence, speculative-verify ticks ``W`` per
sequence, prefill chunks any number.  Every tensor here is an int32 device
tensor so the same object can be the static input block of a CUDA graph.

Parity: reference ``src/tilerl/kv_cache.py:954`` (``BatchKv``); the reference pads
rows to a common width and masks with ``seq_q_lens`` -- here rows are ragged.
"""
from __future__ import annotations

import itertools
import os
from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import numpy as np
import torch

from .ops.ref import KV_BLOCK


@dataclass
class Batch:
    token_ids: torch.Tensor      # [T] int32
    positions: torch.Tensor      # [T] int32 absolute position of each token
    seq_ids: torch.Tensor        # [T] int32 row of the per-sequence arrays
    slot_mapping: torch.Tensor   # [T] int32 physical KV row (block*16+off), -1 = no write
    q_start: torch.Tensor        # [B] int32 first token index of each sequence
    q_len: torch.Tensor          # [B] int32 tokens of each sequence in this tick
    kv_len: torch.Tensor         # [B] int32 KV length after this tick
    state_slots: torch.Tensor    # [B] int32 GDN state slot of each sequence
    block_table: torch.Tensor    # [B, max_blocks] int32
    last_idx: torch.Tensor       # [B] int32 index in [T] of each sequence's last token
    n_seqs: int = 0
    n_tokens: int = 0
    max_q_len: int = 1
    keep_steps: int = 0          # >0: verify tick, keep the GDN state after each token
    sparse: Optional[object] = None   # per-layer selected page lists (sparse KV)
    host_q_len: List[int] = field(default_factory=list)
    host_kv_len: List[int] = field(default_factory=list)
    keep_rows: List[bool] = field(default_factory=list)   # per sequence: store per-token GDN states
    keep_flags: Optional[torch.Tensor] = None             # [B] int32 device copy of keep_rows
    h2d_bytes: int = 0

    @staticmethod
    def build(seqs: Sequence[dict], device, max_blocks: Optional[int] = None,
              keep_steps: int = 0, pad_to: Optional[int] = None) -> "Batch":
        """``seqs``: dicts with ``tokens`` (ids of this tick), ``start`` (position of
        the first), ``blocks`` (physical block ids), ``slot`` (GDN state slot)."""
        mb = max_blocks or max(1, max(len(s["blocks"]) for s in seqs))
        device = torch.device(device)
        ql = [len(s["tokens"]) for s in seqs]
        kl = [int(s["start"]) + n for s, n in zip(seqs, ql)]
        keep = [bool(s.get("keep", False)) and keep_steps > 0 for s in seqs]
        t = sum(ql)
        sizes = [t] * 4 + [len(seqs)] * 6
        total = sum(sizes) + len(seqs) * mb
        on_gpu = device.type == "cuda"
        flat = _pinned(total)[:total] if on_gpu else torch.empty(total, dtype=torch.int32)
        if not (USE_NATIVE and _fill_native(seqs, ql, keep, mb, flat)):
            _fill_python(seqs, ql, kl, keep, mb, flat)
        if on_gpu:
            # one pinned staging block, one async H2D copy for the whole descriptor
            dev = torch.empty(total, dtype=torch.int32, device=device)
            dev.copy_(flat, non_blocking=True)
            _PIN["event"].record()
        else:
            dev = flat
        views, o = [], 0
        for n in sizes:
            views.append(dev[o:o + n])
            o += n
        tbl = dev[o:].view(len(seqs), mb)
        v_ids, v_pos, v_sid, v_smap, v_qs, v_ql, v_kl, v_slots, v_last, v_keep = views
        return Batch(
            token_ids=v_ids, positions=v_pos, seq_ids=v_sid, slot_mapping=v_smap,
            q_start=v_qs, q_len=v_ql, kv_len=v_kl, state_slots=v_slots,
            block_table=tbl, last_idx=v_last, n_seqs=len(seqs), n_tokens=t,
            max_q_len=max(ql), keep_steps=keep_steps, host_q_len=ql, host_kv_len=kl,
            keep_rows=keep, keep_flags=v_keep, h2d_bytes=total * 4,
        )


USE_NATIVE = os.environ.get("TRL_NATIVE_BATCH", "1") != "0"


def _fill_python(seqs, ql, kl, keep, mb: int, flat: torch.Tensor) -> None:
    """Interpreter twin of the native filler (same layout; used when the library is absent)."""
    ids, pos, sid, smap, qs, last, slots = [], [], [], [], [], [], []
    table = torch.zeros(len(seqs), mb, dtype=torch.int32)
    t = 0
    for r, s in enumerate(seqs):
        toks, start, blocks = list(s["tokens"]), int(s["start"]), s["blocks"]
        qs.append(t)
        for j, tok in enumerate(toks):
            p = start + j
            ids.append(tok)
            pos.append(p)
            sid.append(r)
            smap.append(blocks[p // KV_BLOCK] * KV_BLOCK + p % KV_BLOCK)
        t += len(toks)
        last.append(t - 1)
        slots.append(int(s["slot"]))
        if blocks:
            table[r, :len(blocks)] = torch.tensor(blocks, dtype=torch.int32)
    o = 0
    for a in (ids, pos, sid, smap, qs, ql, kl, slots, last, [int(k) for k in keep]):
        flat[o:o + len(a)] = torch.tensor(a, dtype=torch.int32)
        o += len(a)
    flat[o:] = table.reshape(-1)


def _fill_native(seqs, ql, keep, mb: int, flat: torch.Tensor) -> bool:
    """The same descriptor written by ``trl_batch_fill`` of the host runtime (``csrc/runtime.cpp``)
    straight into the staging block.  False when the library is not built."""
    lib = _runtime()
    if lib is None:
        return False
    n = len(seqs)
    tok_off = np.zeros(n + 1, dtype=np.int32)
    np.cumsum(ql, out=tok_off[1:])
    nb = [len(s["blocks"]) for s in seqs]
    blk_off = np.zeros(n + 1, dtype=np.int32)
    np.cumsum(nb, out=blk_off[1:])
    tokens = np.fromiter(itertools.chain.from_iterable(s["tokens"] for s in seqs), dtype=np.int32, count=int(tok_off[-1]))
    blocks = np.fromiter(itertools.chain.from_iterable(s["blocks"] for s in seqs), dtype=np.int32, count=int(blk_off[-1]))
    starts = np.fromiter((int(s["start"]) for s in seqs), dtype=np.int32, count=n)
    slots = np.fromiter((int(s["slot"]) for s in seqs), dtype=np.int32, count=n)
    kp = np.fromiter((int(k) for k in keep), dtype=np.int32, count=n)
    wrote = lib.trl_batch_fill(n, tokens.ctypes.data, tok_off.ctypes.data, starts.ctypes.data, slots.ctypes.data,
                               kp.ctypes.data, blocks.ctypes.data, blk_off.ctypes.data, mb, KV_BLOCK,
                               flat.data_ptr(), flat.numel())
    if wrote == -2:
        raise IndexError("a token of the batch lies beyond its sequence's block list")
    if wrote != flat.numel():
        raise RuntimeError(f"trl_batch_fill wrote {wrote} of {flat.numel()} values")
    return True


_RT = {"lib": None, "tried": False}


def _runtime():
    if not _RT["tried"]:
        _RT["tried"] = True
        try:
            from .ops import native
            if native.loadable():
                _RT["lib"] = native.lib()
                if not hasattr(_RT["lib"], "trl_batch_fill"):
                    _RT["lib"] = None          # a library built before the host runtime existed
        except OSError:
            _RT["lib"] = None
    return _RT["lib"]


_PIN = {"buf": None, "event": None}


def _pinned(n: int) -> torch.Tensor:
    """Grow-only pinned staging buffer; waits for the previous copy out of it."""
    if _PIN["event"] is None:
        _PIN["event"] = torch.cuda.Event()
    else:
        _PIN["event"].synchronize()
    if _PIN["buf"] is None or _PIN["buf"].numel() < n:
        _PIN["buf"] = torch.empty(max(n, 1 << 16), dtype=torch.int32).pin_memory()
    return _PIN["buf"]
