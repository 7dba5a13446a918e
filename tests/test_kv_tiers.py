import os

import torch

from helpers import make_engine, rand_prompts
from tilerl_b200.config import tiny_hybrid
from tilerl_b200.engine import SamplingParams
from tilerl_b200.kv import PrefixStore
from tilerl_b200.kv_tiers import ColdSsdFile, DramSnapshots, HostKvPages, KvBootStore, SpillWriteError


def _page(seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(1, 2, 16, 8, generator=g), torch.randn(1, 2, 16, 8, generator=g)


def test_host_pages_lru_sharing_and_ssd_spill(tmp_path):
    k0, v0 = _page(0)
    nb = k0.numel() * 4 * 2
    cold = ColdSsdFile(str(tmp_path / "spill.bin"), slot_bytes=nb, slots=4)
    host = HostKvPages(budget_bytes=2 * nb, cold=cold)
    keys = [host.demote(*_page(i)) for i in range(4)]
    assert host.demote(*_page(3)) == keys[3] and host.stats["shared"] == 1
    assert len(host.pages) == 2 and host.stats["spilled"] == 2
    for i, key in enumerate(keys):             # promote from host or from the spill file
        k, v = host.promote(key)
        assert torch.equal(k, _page(i)[0]) and torch.equal(v, _page(i)[1])
    assert host.promote("nope") is None
    try:
        cold.put("big", b"x" * (nb + 1))
        assert False
    except SpillWriteError:
        pass
    cold.close()


def test_dram_snapshots_budget():
    d = DramSnapshots(budget_bytes=3000)
    for i in range(4):
        d.put(i, (torch.full((256,), float(i)), torch.zeros(4)))
    assert d.get(0, "cpu") is None and float(d.get(3, "cpu")[0][0]) == 3.0


def test_boot_store_roundtrip_fingerprint_and_crc(tmp_path):
    cfg = tiny_hybrid()
    eng = make_engine(cfg)
    eng.prefix = PrefixStore(eng.kv)
    p = rand_prompts(cfg, 1, 40, seed=9)[0]
    sp = SamplingParams(max_tokens=5)
    cold = eng.generate([p], sp)[0].tokens
    store = KvBootStore(str(tmp_path / "boot"))
    assert store.save(eng) == 1
    fresh = make_engine(cfg, model=eng.model)
    fresh.prefix = PrefixStore(fresh.kv)
    assert store.boot(fresh)["loaded"] == 1
    r = fresh.generate([p], sp)[0]
    assert r.tokens == cold and r.cached_tokens == 32
    other = make_engine(cfg, seed=77)            # different weights: the store is ignored
    other.prefix = PrefixStore(other.kv)
    assert store.boot(other)["skipped_fingerprint"] == 1
    victim = [f for f in os.listdir(tmp_path / "boot") if f.endswith("_0.bin")][0]
    with open(tmp_path / "boot" / victim, "r+b") as f:
        f.write(b"\xff\xff\xff")
    again = make_engine(cfg, model=eng.model)
    again.prefix = PrefixStore(again.kv)
    assert store.boot(again) == dict(loaded=0, skipped_fingerprint=0, corrupt=1)


def test_prefix_store_demotes_to_the_host_tier_and_promotes_on_a_hit():
    """An entry evicted from the device store comes back from host memory with the same tokens,
    KV pages and GDN snapshot -- the request that hits it produces what a cold run produces."""
    from helpers import rand_prompts
    from tilerl_b200.config import tiny_hybrid
    from tilerl_b200.engine import Engine, SamplingParams
    from tilerl_b200.kv import GdnStatePool, PagedKvPool, PrefixStore
    from tilerl_b200.kv_tiers import DramSnapshots, HostKvPages
    from tilerl_b200.models.hybrid import HybridModel
    from tilerl_b200.ops.backend import RefOps
    cfg = tiny_hybrid()
    model = HybridModel.build_random(cfg, seed=1)
    kv = PagedKvPool(cfg, 64, dtype=torch.float32)
    st = GdnStatePool(cfg, 6, ring_dtype=torch.float32)
    store = PrefixStore(kv, max_entries=1, host=HostKvPages(1 << 26), dram=DramSnapshots(1 << 26))
    eng = Engine(model, RefOps(), kv, st, prefix_store=store)
    a, b = rand_prompts(cfg, 2, 40)
    sp = SamplingParams(max_tokens=5)
    cold = eng.generate([a], sp)[0]
    eng.generate([b], sp)                          # max_entries = 1: publishing b evicts a -> host tier
    assert store.demotions >= 1 and len(store.cold) >= 1
    warm = eng.generate([a], sp)[0]
    assert store.promotions == 1
    assert warm.tokens == cold.tokens and warm.cached_tokens == 32


def test_clear_drops_cold_tiers_too_so_a_weight_change_cannot_serve_stale_kv():
    """``Engine.invalidate_weights`` clears the prefix store: an entry that had been demoted to host
    memory must not be promoted afterwards (it was computed with the old weights), and clearing
    must not copy anything to the host on the way."""
    from helpers import rand_prompts
    from tilerl_b200.config import tiny_hybrid
    from tilerl_b200.engine import Engine, SamplingParams
    from tilerl_b200.kv import GdnStatePool, PagedKvPool, PrefixStore
    from tilerl_b200.kv_tiers import DramSnapshots, HostKvPages
    from tilerl_b200.models.hybrid import HybridModel
    from tilerl_b200.ops.backend import RefOps
    cfg = tiny_hybrid()
    model = HybridModel.build_random(cfg, seed=1)
    kv = PagedKvPool(cfg, 64, dtype=torch.float32)
    st = GdnStatePool(cfg, 6, ring_dtype=torch.float32)
    host, dram = HostKvPages(1 << 26), DramSnapshots(1 << 26)
    store = PrefixStore(kv, max_entries=1, host=host, dram=dram)
    eng = Engine(model, RefOps(), kv, st, prefix_store=store)
    a, b = rand_prompts(cfg, 2, 40)
    sp = SamplingParams(max_tokens=3)
    eng.generate([a], sp)
    eng.generate([b], sp)                          # a is now cold (host pages + DRAM snapshot), b is warm
    assert len(store.cold) == 1 and len(store.entries) == 1
    demotions, free_before = store.demotions, None
    eng.invalidate_weights()
    assert len(store.entries) == 0 and len(store.cold) == 0
    assert store.demotions == demotions            # nothing was copied out while clearing
    assert len(host.pages) == 0 and len(dram.items) == 0 and dram.bytes == 0
    assert kv.used_blocks == 0
    misses = store.misses
    again = eng.generate([a], sp)[0]
    assert again.cached_tokens == 0 and store.misses == misses + 1 and store.promotions == 0


def test_refcount_calls_survive_python_optimised_mode(tmp_path):
    """The native incref / release calls are statements of their own (never the operand of an
    ``assert``): under ``python -O`` a shared prefix block keeps its references."""
    import subprocess
    import sys
    code = (
        "import torch\n"
        "from tilerl_b200.config import tiny_hybrid\n"
        "from tilerl_b200.kv import PagedKvPool\n"
        "kv = PagedKvPool(tiny_hybrid(), 8, dtype=torch.float32)\n"
        "b = kv.alloc_block(); free = kv.free_blocks\n"
        "kv.incref(b); kv.release(b)\n"
        "assert_free = kv.free_blocks\n"
        "kv.release(b)\n"
        "print(free, assert_free, kv.free_blocks)\n")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = subprocess.run([sys.executable, "-O", "-c", code], capture_output=True, text=True, cwd=root,
                         env={**os.environ, "PYTHONPATH": root})
    assert out.returncode == 0, out.stderr
    free, mid, end = map(int, out.stdout.split())
    assert mid == free and end == free + 1
