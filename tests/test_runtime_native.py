"""Host runtime (csrc/runtime.cpp): the C++ block allocator and batch filler against their
Python twins."""
import random

import pytest
import torch

from tilerl_b200 import batch as B
from tilerl_b200.config import tiny_hybrid
from tilerl_b200.kv import PagedKvPool, PoolExhausted
from tilerl_b200.ops import native

needs_lib = pytest.mark.skipif(not native.loadable(), reason="library not built")


def _random_seqs(rng, n):
    seqs, blk = [], 1
    for i in range(n):
        start, nt = rng.randint(0, 100), rng.randint(1, 40)
        nb = (start + nt + 15) // 16 + rng.randint(0, 2)
        seqs.append(dict(tokens=[rng.randint(0, 999) for _ in range(nt)], start=start,
                         blocks=list(range(blk, blk + nb)), slot=i + 1, keep=bool(i % 2)))
        blk += nb
    return seqs


@needs_lib
def test_native_batch_filler_equals_python(monkeypatch):
    rng = random.Random(0)
    fields = ("token_ids", "positions", "seq_ids", "slot_mapping", "q_start", "q_len", "kv_len", "state_slots",
              "block_table", "last_idx", "keep_flags")
    for trial in range(25):
        seqs = _random_seqs(rng, rng.randint(1, 9))
        kw = dict(keep_steps=trial % 2, max_blocks=None if trial % 3 else 12)
        monkeypatch.setattr(B, "USE_NATIVE", True)
        a = B.Batch.build(seqs, "cpu", **kw)
        monkeypatch.setattr(B, "USE_NATIVE", False)
        b = B.Batch.build(seqs, "cpu", **kw)
        for f in fields:
            assert torch.equal(getattr(a, f), getattr(b, f)), f
        assert (a.n_tokens, a.max_q_len, a.host_kv_len, a.keep_rows) == (b.n_tokens, b.max_q_len, b.host_kv_len, b.keep_rows)


@needs_lib
def test_native_batch_filler_rejects_a_token_beyond_its_blocks(monkeypatch):
    monkeypatch.setattr(B, "USE_NATIVE", True)
    with pytest.raises(IndexError):
        B.Batch.build([dict(tokens=[1] * 20, start=0, blocks=[3], slot=1)], "cpu")


@pytest.mark.parametrize("native_on", [True, False])
def test_block_allocator_refcounts(native_on, monkeypatch):
    if native_on and not native.loadable():
        pytest.skip("library not built")
    monkeypatch.setenv("TRL_NATIVE_PAGER", "1" if native_on else "0")
    pool = PagedKvPool(tiny_hybrid(), 6, dtype=torch.float32)
    assert (pool._pager is not None) == native_on
    assert pool.free_blocks == 5 and pool.used_blocks == 0
    got = [pool.alloc_block() for _ in range(5)]
    assert got == [1, 2, 3, 4, 5]
    with pytest.raises(PoolExhausted):
        pool.alloc_block()
    pool.incref(3)
    pool.release(3)
    assert pool.free_blocks == 0 and pool.ref[3] == 1
    pool.release(3)
    assert pool.free_blocks == 1 and pool.ref[3] == 0 and pool.ref[0] == 1
    assert pool.alloc_block() == 3
    with pytest.raises(AssertionError):
        pool.release(0)
    pool.release(5)
    with pytest.raises(AssertionError):
        pool.release(5)
    with pytest.raises(AssertionError):
        pool.incref(5)
    assert pool.used_blocks == 4
