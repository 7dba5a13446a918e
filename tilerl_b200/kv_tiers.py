"""KV tiers below the device pool: pinned host pages, an SSD spill file, DRAM snapshots of
GDN state, and an on-disk cold-start store.

* :class:`HostKvPages` -- byte-budgeted LRU of demoted KV pages in (pinned) host memory,
  keyed by page *content hash* so identical pages from different requests share one blob.
* :class:`ColdSsdFile` -- fixed-slot spill file (mmap) behind the host tier; a failed write
  raises :class:`SpillWriteError` and the page simply stays un-demoted.
* :class:`DramSnapshots` -- LRU of GDN state snapshots demoted from the prefix store.
* :class:`KvBootStore` -- persist prefix entries across restarts: a JSON manifest, one blob
  per page with a CRC32, and the weights' fingerprint (a store written for other weights is
  ignored, a corrupted page is dropped).

Parity: reference ``src/tilerl/kv_tiers.py`` -- ``ColdSsdFile:115``, ``HostKvPages:431``,
``DramSnapshots:1007``, ``KvBootStore:1114`` (``save:1214``, ``boot:1308``).
"""
from __future__ import annotations

import hashlib
import json
import mmap
import os
import zlib
from collections import OrderedDict
from typing import Dict, List, Optional, Tuple

import torch


class SpillWriteError(IOError):
    pass


def page_key(k: torch.Tensor, v: torch.Tensor) -> str:
    h = hashlib.blake2b(digest_size=16)
    h.update(k.contiguous().view(torch.uint8).cpu().numpy().tobytes())
    h.update(v.contiguous().view(torch.uint8).cpu().numpy().tobytes())
    return h.hexdigest()


class ColdSsdFile:
    def __init__(self, path: str, slot_bytes: int, slots: int):
        self.path, self.slot_bytes, self.slots = path, slot_bytes, slots
        os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
        with open(path, "wb") as f:
            f.truncate(slot_bytes * slots)
        self.f = open(path, "r+b")
        self.mm = mmap.mmap(self.f.fileno(), slot_bytes * slots)
        self.free = list(range(slots - 1, -1, -1))
        self.index: Dict[str, int] = {}

    def put(self, key: str, blob: bytes) -> bool:
        if key in self.index:
            return True
        if len(blob) > self.slot_bytes:
            raise SpillWriteError(f"page of {len(blob)} B exceeds slot of {self.slot_bytes} B")
        if not self.free:
            return False
        s = self.free.pop()
        try:
            self.mm[s * self.slot_bytes:s * self.slot_bytes + len(blob)] = blob
        except (ValueError, OSError) as e:
            self.free.append(s)
            raise SpillWriteError(str(e)) from e
        self.index[key] = s
        return True

    def get(self, key: str, nbytes: int) -> Optional[bytes]:
        s = self.index.get(key)
        return None if s is None else bytes(self.mm[s * self.slot_bytes:s * self.slot_bytes + nbytes])

    def drop(self, key: str) -> None:
        s = self.index.pop(key, None)
        if s is not None:
            self.free.append(s)

    def close(self) -> None:
        self.mm.close()
        self.f.close()


class HostKvPages:
    def __init__(self, budget_bytes: int, pin: bool = False, cold: Optional[ColdSsdFile] = None):
        self.budget, self.pin, self.cold = budget_bytes, pin, cold
        self.pages: "OrderedDict[str, Tuple[torch.Tensor, torch.Tensor, int]]" = OrderedDict()
        self.bytes = 0
        self.stats = dict(demoted=0, promoted=0, shared=0, spilled=0, dropped=0, spill_errors=0)
        self._shapes: Dict[str, Tuple[tuple, torch.dtype]] = {}

    def _host(self, t: torch.Tensor) -> torch.Tensor:
        h = t.detach().to("cpu", copy=True)
        return h.pin_memory() if self.pin and torch.cuda.is_available() else h

    def demote(self, k: torch.Tensor, v: torch.Tensor) -> str:
        """Store a page ([layers, hkv, 16, D] each); returns its content key."""
        key = page_key(k, v)
        if key in self.pages:
            kk, vv, rc = self.pages[key]
            self.pages[key] = (kk, vv, rc + 1)
            self.pages.move_to_end(key)
            self.stats["shared"] += 1
            return key
        kk, vv = self._host(k), self._host(v)
        nb = kk.numel() * kk.element_size() * 2
        self.pages[key] = (kk, vv, 1)
        self.bytes += nb
        self.stats["demoted"] += 1
        while self.bytes > self.budget and len(self.pages) > 1:
            self._evict_one()
        return key

    def _evict_one(self) -> None:
        key, (kk, vv, _) = self.pages.popitem(last=False)
        self.bytes -= kk.numel() * kk.element_size() * 2
        if self.cold is not None:
            try:
                blob = kk.view(torch.uint8).numpy().tobytes() + vv.view(torch.uint8).numpy().tobytes()
                if self.cold.put(key, blob):
                    self.stats["spilled"] += 1
                    self._shapes[key] = (tuple(kk.shape), kk.dtype)
                    return
            except SpillWriteError:
                self.stats["spill_errors"] += 1
        self.stats["dropped"] += 1

    def promote(self, key: str) -> Optional[Tuple[torch.Tensor, torch.Tensor]]:
        ent = self.pages.get(key)
        if ent is not None:
            self.pages.move_to_end(key)
            self.stats["promoted"] += 1
            return ent[0], ent[1]
        if self.cold is not None and key in self.cold.index:
            shape, dtype = self._shapes[key]
            n = 1
            for s in shape:
                n *= s
            nb = n * torch.empty(0, dtype=dtype).element_size()
            blob = self.cold.get(key, 2 * nb)
            k = torch.frombuffer(bytearray(blob[:nb]), dtype=torch.uint8).view(dtype).view(shape)
            v = torch.frombuffer(bytearray(blob[nb:]), dtype=torch.uint8).view(dtype).view(shape)
            self.stats["promoted"] += 1
            return k, v
        return None

    def release(self, key: str) -> None:
        ent = self.pages.get(key)
        if ent is None:
            return
        kk, vv, rc = ent
        if rc > 1:
            self.pages[key] = (kk, vv, rc - 1)
        else:
            del self.pages[key]
            self.bytes -= kk.numel() * kk.element_size() * 2


class DramSnapshots:
    """LRU of GDN state snapshots (state planes + conv ring) in host memory."""

    def __init__(self, budget_bytes: int):
        self.budget = budget_bytes
        self.items: "OrderedDict[int, Tuple[torch.Tensor, torch.Tensor]]" = OrderedDict()
        self.bytes = 0

    @staticmethod
    def _nbytes(s) -> int:
        return sum(t.numel() * t.element_size() for t in s)

    def put(self, key: int, snap: Tuple[torch.Tensor, torch.Tensor]) -> None:
        host = tuple(t.detach().to("cpu", copy=True) for t in snap)
        self.items[key] = host
        self.bytes += self._nbytes(host)
        while self.bytes > self.budget and len(self.items) > 1:
            _, old = self.items.popitem(last=False)
            self.bytes -= self._nbytes(old)

    def get(self, key: int, device) -> Optional[Tuple[torch.Tensor, torch.Tensor]]:
        s = self.items.get(key)
        if s is None:
            return None
        self.items.move_to_end(key)
        return tuple(t.to(device) for t in s)

    def drop(self, key: int) -> None:
        s = self.items.pop(key, None)
        if s is not None:
            self.bytes -= self._nbytes(s)


def weights_fingerprint(model) -> str:
    """Cheap identity of the served weights: shapes plus a sample of bytes of every tensor."""
    h = hashlib.blake2b(digest_size=16)
    for k in sorted(model.params):
        v = model.params[k]
        t = v.wq if hasattr(v, "wq") else (v.w8 if hasattr(v, "w8") else v)
        h.update(k.encode())
        h.update(str(tuple(t.shape)).encode())
        flat = t.reshape(-1)[:: max(1, t.numel() // 64)][:64]
        h.update(flat.contiguous().view(torch.uint8).cpu().numpy().tobytes())
    return h.hexdigest()


class KvBootStore:
    """Persist prefix-store entries (token ids, KV pages, GDN snapshot) for a warm restart."""

    def __init__(self, root: str):
        self.root = root
        os.makedirs(root, exist_ok=True)

    def save(self, engine) -> int:
        store, pool = engine.prefix, engine.kv
        entries = []
        for key, e in getattr(store, "entries", {}).items():
            pages = []
            for i, b in enumerate(e.blocks):
                k, v = pool.read_block(b)
                blob = k.contiguous().view(torch.uint8).cpu().numpy().tobytes() + \
                    v.contiguous().view(torch.uint8).cpu().numpy().tobytes()
                fn = f"{key:x}_{i}.bin"
                with open(os.path.join(self.root, fn + ".tmp"), "wb") as f:
                    f.write(blob)
                os.replace(os.path.join(self.root, fn + ".tmp"), os.path.join(self.root, fn))
                pages.append({"file": fn, "crc": zlib.crc32(blob), "nbytes": len(blob)})
            snap_fn = None
            if e.snapshot is not None:
                snap_fn = f"{key:x}_state.pt"
                torch.save([t.cpu() for t in e.snapshot], os.path.join(self.root, snap_fn))
            entries.append({"tokens": list(e.tokens), "pages": pages, "snapshot": snap_fn})
        man = {"fingerprint": weights_fingerprint(engine.model), "entries": entries,
               "page_shape": list(pool.k[:, 0].shape), "dtype": str(pool.k.dtype)}
        with open(os.path.join(self.root, "manifest.json.tmp"), "w") as f:
            json.dump(man, f)
        os.replace(os.path.join(self.root, "manifest.json.tmp"), os.path.join(self.root, "manifest.json"))
        return len(entries)

    def boot(self, engine) -> Dict[str, int]:
        """Re-insert stored entries into the engine's prefix store.  Returns counters."""
        out = dict(loaded=0, skipped_fingerprint=0, corrupt=0)
        mp = os.path.join(self.root, "manifest.json")
        if not os.path.exists(mp):
            return out
        with open(mp) as f:
            man = json.load(f)
        if man.get("fingerprint") != weights_fingerprint(engine.model):
            out["skipped_fingerprint"] = len(man.get("entries", []))
            return out
        pool = engine.kv
        shape = tuple(man["page_shape"])
        for e in man["entries"]:
            blobs, ok = [], True
            for pg in e["pages"]:
                try:
                    with open(os.path.join(self.root, pg["file"]), "rb") as f:
                        blob = f.read()
                except OSError:
                    ok = False
                    break
                if len(blob) != pg["nbytes"] or zlib.crc32(blob) != pg["crc"]:
                    ok = False
                    break
                blobs.append(blob)
            if not ok or pool.free_blocks < len(blobs):
                out["corrupt"] += 0 if ok else 1
                continue
            blocks = []
            for blob in blobs:
                half = len(blob) // 2
                b = pool.alloc_block()
                k = torch.frombuffer(bytearray(blob[:half]), dtype=torch.uint8).view(pool.k.dtype).view(shape)
                v = torch.frombuffer(bytearray(blob[half:]), dtype=torch.uint8).view(pool.k.dtype).view(shape)
                pool.write_block(b, k.to(pool.k.device), v.to(pool.k.device))
                blocks.append(b)
            snap = None
            if e["snapshot"]:
                snap = tuple(t.to(engine.states.states.device)
                             for t in torch.load(os.path.join(self.root, e["snapshot"]), weights_only=False))
            engine.prefix.insert(e["tokens"], blocks, snap)
            for b in blocks:            # the store holds its own references now
                pool.release(b)
            out["loaded"] += 1
        return out
