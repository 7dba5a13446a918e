"""Device-resident sequence state: paged KV pool, GDN state pool, prefix store.

* :class:`PagedKvPool` -- ``k/v [attn_layers, blocks, hkv, 16, D]`` (bf16, or e4m3
  with one fp32 scale per (block, head, token)); free list + refcounts; block 0
  is a reserved pad page that CUDA-graph padding rows write into.
* :class:`GdnStatePool` -- ``states [slots, gdn_layers, planes, nv, dk, dv]`` fp32
  and a raw-qkv ring ``[slots, gdn_layers, R, C]`` indexed by ``position % R``.
  ``planes > 1`` keeps the state after each token of a speculative-verify tick;
  ``cur[slot]`` names the live plane, so adopting "the state after n accepted
  tokens" is one int32 write instead of a 144 MiB copy, and the conv window
  needs no rollback at all because the ring is addressed by absolute position.
* :class:`PrefixStore` -- rolling-hash cache of whole 16-token blocks; an entry
  owns refcounted block ids *and* a GDN snapshot taken at the same boundary
  (a hybrid model needs both to resume).

Parity: reference ``src/tilerl/kv_cache.py`` -- ``PagedKvPool:53``,
``LinearStatePool:533`` (double-buffered windows + ``step_states``),
``PrefixStore:694``.
"""
from __future__ import annotations

import ctypes
import os
from collections import OrderedDict
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from .config import ModelConfig
from .ops.ref import KV_BLOCK

RING = 16  # conv ring rows; >= spec width + conv taps


class PoolExhausted(RuntimeError):
    pass


def _native_pager(num_blocks: int):
    """``(lib, handle)`` of a C++ block allocator (``csrc/runtime.cpp``), or None when the library
    is not built or ``TRL_NATIVE_PAGER=0``."""
    if os.environ.get("TRL_NATIVE_PAGER", "1") == "0":
        return None
    try:
        from .ops import native
        if not native.loadable():
            return None
        lib = native.lib()
        if not hasattr(lib, "trl_pager_create"):
            return None
        h = lib.trl_pager_create(int(num_blocks))
        return (lib, ctypes.c_void_p(h)) if h else None
    except OSError:
        return None


class PagedKvPool:
    def __init__(self, cfg: ModelConfig, num_blocks: int, device="cpu",
                 dtype=torch.bfloat16, fp8: bool = False, n_kv_heads: Optional[int] = None):
        self.cfg = cfg
        self.num_blocks = int(num_blocks)
        self.hkv = n_kv_heads or cfg.n_kv_heads
        self.fp8 = fp8
        shape = (max(1, cfg.n_attn_layers), self.num_blocks, self.hkv, KV_BLOCK, cfg.head_dim)
        store = torch.float8_e4m3fn if fp8 else dtype
        self.k = torch.zeros(shape, dtype=store, device=device)
        self.v = torch.zeros(shape, dtype=store, device=device)
        if fp8:
            self.k_scale = torch.ones(shape[:-1], dtype=torch.float32, device=device)
            self.v_scale = torch.ones(shape[:-1], dtype=torch.float32, device=device)
        self._pager = _native_pager(self.num_blocks)     # C++ free list + refcounts when the library is built
        if self._pager is None:
            self._ref = [0] * self.num_blocks
            self._ref[0] = 1  # pad page, never handed out
            self._free = list(range(self.num_blocks - 1, 0, -1))

    def __del__(self):
        pg = getattr(self, "_pager", None)
        if pg is not None:
            self._pager = None
            try:
                pg[0].trl_pager_destroy(pg[1])
            except Exception:  # noqa: BLE001 - interpreter shutdown: the library may be gone already
                pass

    # ---- allocator -----------------------------------------------------------
    @property
    def ref(self) -> List[int]:
        """Reference count of every block (a copy when the native allocator holds them)."""
        if self._pager is None:
            return self._ref
        lib, h = self._pager
        buf = (ctypes.c_int32 * self.num_blocks)()
        lib.trl_pager_refs(h, buf, self.num_blocks)
        return list(buf)

    @property
    def free_blocks(self) -> int:
        if self._pager is not None:
            return self._pager[0].trl_pager_free_count(self._pager[1])
        return len(self._free)

    @property
    def used_blocks(self) -> int:
        return self.num_blocks - 1 - self.free_blocks

    def alloc_block(self) -> int:
        if self._pager is not None:
            b = self._pager[0].trl_pager_alloc(self._pager[1])
            if b < 0:
                raise PoolExhausted("KV pool has no free block")
            return b
        if not self._free:
            raise PoolExhausted("KV pool has no free block")
        b = self._free.pop()
        self._ref[b] = 1
        return b

    def incref(self, b: int) -> None:
        if self._pager is not None:
            rc = self._pager[0].trl_pager_incref(self._pager[1], int(b))   # the call itself, never inside an assert
            if rc <= 0:
                raise AssertionError(f"incref of free block {b}")
            return
        assert self._ref[b] > 0, f"incref of free block {b}"
        self._ref[b] += 1

    def release(self, b: int) -> None:
        if self._pager is not None:
            rc = self._pager[0].trl_pager_release(self._pager[1], int(b))
            if rc < 0:
                raise AssertionError(f"release of free block {b}")
            return
        assert b != 0 and self._ref[b] > 0, f"release of free block {b}"
        self._ref[b] -= 1
        if self._ref[b] == 0:
            self._free.append(b)

    def block_bytes(self) -> int:
        per = self.hkv * KV_BLOCK * self.cfg.head_dim * self.k.element_size() * 2
        if self.fp8:
            per += self.hkv * KV_BLOCK * 4 * 2
        return per * max(1, self.cfg.n_attn_layers)

    def layer(self, attn_idx: int) -> Tuple[torch.Tensor, torch.Tensor]:
        return self.k[attn_idx], self.v[attn_idx]

    # ---- host tier hooks -------------------------------------------------------
    def read_block(self, b: int) -> Tuple[torch.Tensor, torch.Tensor]:
        if self.fp8:     # tiers move the dequantised page; the scales are re-derived on the way back
            return (self.k[:, b].float() * self.k_scale[:, b].unsqueeze(-1),
                    self.v[:, b].float() * self.v_scale[:, b].unsqueeze(-1))
        return self.k[:, b].clone(), self.v[:, b].clone()

    def write_block(self, b: int, k: torch.Tensor, v: torch.Tensor) -> None:
        if self.fp8:
            from .formats import quantize_kv_fp8
            k8, ks = quantize_kv_fp8(k.float())
            v8, vs = quantize_kv_fp8(v.float())
            self.k[:, b].copy_(k8), self.v[:, b].copy_(v8)
            self.k_scale[:, b].copy_(ks), self.v_scale[:, b].copy_(vs)
            return
        self.k[:, b].copy_(k)
        self.v[:, b].copy_(v)


class GdnStatePool:
    def __init__(self, cfg: ModelConfig, num_slots: int, device="cpu", planes: int = 1,
                 ring_dtype=torch.bfloat16, n_v_heads: Optional[int] = None,
                 n_k_heads: Optional[int] = None):
        self.cfg = cfg
        self.num_slots = int(num_slots)
        self.planes = int(planes)
        self.nv = n_v_heads or cfg.gdn_v_heads
        self.nk = n_k_heads or cfg.gdn_k_heads
        ng = max(1, cfg.n_gdn_layers)
        d = max(1, cfg.gdn_head_dim)
        self.conv_dim = 2 * self.nk * d + self.nv * d
        self.states = torch.zeros(self.num_slots, ng, self.planes, max(1, self.nv), d, d,
                                  dtype=torch.float32, device=device)
        self.ring = torch.zeros(self.num_slots, ng, RING, max(1, self.conv_dim),
                                dtype=ring_dtype, device=device)
        self.cur = torch.zeros(self.num_slots, dtype=torch.int32, device=device)
        self._free = list(range(self.num_slots - 1, 0, -1))  # slot 0 = pad slot

    @property
    def free_slots(self) -> int:
        return len(self._free)

    def alloc_slot(self) -> int:
        if not self._free:
            raise PoolExhausted("GDN state pool has no free slot")
        s = self._free.pop()
        self.states[s].zero_()
        self.ring[s].zero_()
        self.cur[s] = 0
        return s

    def release(self, s: int) -> None:
        assert s != 0 and s not in self._free
        self._free.append(s)

    def slot_bytes(self) -> int:
        return (self.states[0].numel() * 4 + self.ring[0].numel() * self.ring.element_size())

    def live_state(self, slot: int, gdn_idx: int) -> torch.Tensor:
        return self.states[slot, gdn_idx, int(self.cur[slot])]

    def select_step(self, slot: int, step: int) -> None:
        """Adopt the state stored after token ``step`` (0-based) of the last verify tick."""
        self.cur[slot] = step

    def snapshot(self, slot: int) -> Tuple[torch.Tensor, torch.Tensor]:
        return (self.states[slot, :, int(self.cur[slot])].clone(), self.ring[slot].clone())

    def restore(self, slot: int, snap: Tuple[torch.Tensor, torch.Tensor]) -> None:
        self.states[slot, :, 0].copy_(snap[0])
        self.cur[slot] = 0
        self.ring[slot].copy_(snap[1])


# ---- prefix store ------------------------------------------------------------------
_MASK = (1 << 61) - 1


def rolling_hash(prev: int, tokens: Sequence[int]) -> int:
    h = prev
    for t in tokens:
        h = (h * 1000003 + int(t) + 1) & _MASK
    return h


@dataclass
class PrefixHit:
    n_tokens: int
    blocks: List[int]
    snapshot: Optional[Tuple[torch.Tensor, torch.Tensor]]


@dataclass
class _Entry:
    tokens: Tuple[int, ...]
    blocks: List[int]
    snapshot: Optional[Tuple[torch.Tensor, torch.Tensor]]
    state_bytes: int = 0


class NoPrefixStore:
    """Null object: never hits, never stores (RL rollouts use this so weight
    updates cannot be served stale KV)."""
    hits = misses = evictions = 0

    def lookup(self, tokens):  # noqa: D401
        return None

    def insert(self, tokens, blocks, snapshot):
        return False

    def evict_until_free(self, need: int) -> int:
        return 0

    def clear(self) -> None:
        pass

    def __len__(self) -> int:
        return 0


@dataclass
class _Cold:
    """An evicted entry whose pages live in the host tier (content keys) and whose GDN snapshot
    lives in the DRAM tier."""
    tokens: Tuple[int, ...]
    page_keys: List[str]
    has_snapshot: bool


class PrefixStore:
    def __init__(self, pool: PagedKvPool, max_entries: int = 256,
                 max_state_bytes: int = 1 << 30, host=None, dram=None, max_cold: int = 1024):
        """``host`` (``kv_tiers.HostKvPages``) and ``dram`` (``kv_tiers.DramSnapshots``): evicted
        entries are demoted there instead of being dropped, and promoted back on a later hit."""
        self.pool = pool
        self.max_entries = max_entries
        self.max_state_bytes = max_state_bytes
        self.entries: "OrderedDict[int, _Entry]" = OrderedDict()
        self.state_bytes = 0
        self.hits = self.misses = self.evictions = 0
        self.host, self.dram, self.max_cold = host, dram, max_cold
        self.cold: "OrderedDict[int, _Cold]" = OrderedDict()
        self.promotions = self.demotions = 0

    def __len__(self) -> int:
        return len(self.entries)

    def insert(self, tokens: Sequence[int], blocks: Sequence[int], snapshot) -> bool:
        """Publish the prefix ``tokens`` (whole blocks only) with the GDN snapshot
        taken right after its last token."""
        n = len(tokens) - len(tokens) % KV_BLOCK
        if n == 0 or len(blocks) < n // KV_BLOCK:
            return False
        toks = tuple(int(t) for t in tokens[:n])
        key = rolling_hash(0, toks)
        if key in self.entries:
            self.entries.move_to_end(key)
            return False
        blks = list(blocks[: n // KV_BLOCK])
        for b in blks:
            self.pool.incref(b)
        sb = 0 if snapshot is None else sum(t.numel() * t.element_size() for t in snapshot)
        self.entries[key] = _Entry(toks, blks, snapshot, sb)
        self.state_bytes += sb
        while len(self.entries) > self.max_entries or self.state_bytes > self.max_state_bytes:
            if not self._evict_one():
                break
        return True

    def lookup(self, tokens: Sequence[int]) -> Optional[PrefixHit]:
        """Longest stored prefix of ``tokens`` that leaves at least one token to
        run (the last prompt token must go through the model to produce logits)."""
        limit = (len(tokens) - 1) // KV_BLOCK
        hashes, h = [], 0
        for i in range(limit):
            h = rolling_hash(h, tokens[i * KV_BLOCK:(i + 1) * KV_BLOCK])
            hashes.append(h)
        for i in range(limit - 1, -1, -1):
            e = self.entries.get(hashes[i])
            if e is None:
                continue
            n = (i + 1) * KV_BLOCK
            if e.tokens != tuple(int(t) for t in tokens[:n]):
                continue  # hash collision: verified compare refuses it
            self.entries.move_to_end(hashes[i])
            for b in e.blocks:
                self.pool.incref(b)
            self.hits += 1
            return PrefixHit(n, list(e.blocks), e.snapshot)
        for i in range(limit - 1, -1, -1):          # colder: pages in host memory / on SSD
            hit = self._promote(hashes[i], tokens[:(i + 1) * KV_BLOCK])
            if hit is not None:
                self.hits += 1
                return hit
        self.misses += 1
        return None

    def _promote(self, key: int, tokens: Sequence[int]) -> Optional[PrefixHit]:
        c = self.cold.get(key)
        if c is None or c.tokens != tuple(int(t) for t in tokens):
            return None
        if self.pool.free_blocks < len(c.page_keys):
            self.evict_until_free(len(c.page_keys))
            if self.pool.free_blocks < len(c.page_keys):
                return None
        pages = [self.host.promote(k) for k in c.page_keys]
        snap = self.dram.get(key, self.pool.k.device) if (c.has_snapshot and self.dram is not None) else None
        if any(p is None for p in pages) or (c.has_snapshot and snap is None):
            del self.cold[key]                      # a tier dropped part of it: the entry is gone
            return None
        blocks = []
        for k, v in pages:
            b = self.pool.alloc_block()
            self.pool.write_block(b, k.to(self.pool.k.device), v.to(self.pool.k.device))
            blocks.append(b)
        del self.cold[key]
        sb = 0 if snap is None else sum(t.numel() * t.element_size() for t in snap)
        self.entries[key] = _Entry(c.tokens, blocks, snap, sb)     # the store keeps the allocation's reference
        self.state_bytes += sb
        self.promotions += 1
        for b in blocks:
            self.pool.incref(b)                     # the requester's reference
        return PrefixHit(len(c.tokens), list(blocks), snap)

    def _evict_one(self) -> bool:
        if not self.entries:
            return False
        key, e = self.entries.popitem(last=False)
        if self.host is not None:
            keys = [self.host.demote(*self.pool.read_block(b)) for b in e.blocks]
            if e.snapshot is not None and self.dram is not None:
                self.dram.put(key, e.snapshot)
            self.cold[key] = _Cold(e.tokens, keys, e.snapshot is not None and self.dram is not None)
            self.demotions += 1
            while len(self.cold) > self.max_cold:
                _, old = self.cold.popitem(last=False)
                for k in old.page_keys:
                    self.host.release(k)
        for b in e.blocks:
            self.pool.release(b)
        self.state_bytes -= e.state_bytes
        self.evictions += 1
        return True

    def evict_until_free(self, need: int) -> int:
        n = 0
        while self.pool.free_blocks < need and self._evict_one():
            n += 1
        return n

    def clear(self) -> None:
        """Drop every entry, warm and cold, WITHOUT demoting: the store is cleared when the weights
        changed, and KV pages or GDN snapshots computed with the old weights must not come back from
        a host / DRAM tier on a later lookup."""
        while self.entries:
            _, e = self.entries.popitem(last=False)
            for b in e.blocks:
                self.pool.release(b)
            self.state_bytes -= e.state_bytes
            self.evictions += 1
        while self.cold:
            key, c = self.cold.popitem(last=False)
            if self.host is not None:
                for k in c.page_keys:
                    self.host.release(k)
            if c.has_snapshot and self.dram is not None:
                self.dram.drop(key)
