"""Context-parallel gates on CPU ranks (gloo): a zigzag-split forward/backward over 2 ranks must
reproduce the single-rank logits and gradients; dropping the conv halo must break it."""
import pytest
import torch

from world_helpers import run_world

T_LEN = 32


def _setup():
    from tilerl_b200.config import tiny_hybrid
    from tilerl_b200.models.hybrid import HybridModel
    cfg = tiny_hybrid()
    model = HybridModel.build_random(cfg, seed=5, keep_master=True)
    g = torch.Generator().manual_seed(3)
    ids = torch.randint(0, cfg.vocab, (2, T_LEN), generator=g)
    wts = torch.rand(2, T_LEN, generator=g) / (2 * T_LEN)
    return cfg, model, ids, wts


def _single():
    from tilerl_b200 import tape as T
    cfg, model, ids, wts = _setup()
    tr = model.trainable("full")
    tp = T.Tape()
    tp.watch(*tr.values())
    logits = model.forward_dense(tp, ids)
    loss = T.cross_entropy(tp, logits, torch.roll(ids, -1, 1), wts)
    grads = tp.backward(loss)
    return logits.numpy().copy(), {n: grads[id(t)].numpy().copy() for n, t in tr.items() if id(t) in grads}


def _cp_rank(rank, world, halo):
    import torch.distributed as dist
    from tilerl_b200 import tape as T
    from tilerl_b200.parallel.cp import CPContext, positions_for, split_zigzag
    cfg, model, ids, wts = _setup()
    cp = CPContext(dist.group.WORLD, world, rank, halo=halo)
    pos = positions_for(T_LEN, cp)
    tr = model.trainable("full")
    tp = T.Tape()
    tp.watch(*tr.values())
    logits = model.forward_dense(tp, split_zigzag(ids, world, rank), positions=pos, cp=cp)
    targets = split_zigzag(torch.roll(ids, -1, 1), world, rank)
    loss = T.cross_entropy(tp, logits, targets, split_zigzag(wts, world, rank))
    grads = tp.backward(loss)
    out = {}
    for n, t in sorted(tr.items()):
        g = grads.get(id(t))
        g = torch.zeros_like(t, dtype=torch.float32) if g is None else g.float().contiguous()
        dist.all_reduce(g)                       # every rank saw part of the tokens
        out[n] = g.numpy().copy()
    return logits.numpy().copy(), out


def _rel(a, b):
    a, b = torch.from_numpy(a).double(), torch.from_numpy(b).double()
    return float((a - b).norm() / (b.norm() + 1e-30))


@pytest.mark.parametrize("world", [2, 4])
def test_cp_forward_backward_equals_single_rank(world):
    from tilerl_b200.parallel.cp import merge_zigzag
    want_logits, want_grads = _single()
    got = run_world(world, _cp_rank, True)
    logits = merge_zigzag([torch.from_numpy(g[0]) for g in got]).numpy()
    assert _rel(logits, want_logits) < 1e-4
    for n, g in want_grads.items():
        assert _rel(got[0][1][n], g) < 2e-3, n


def test_cp_negative_control_without_halo():
    from tilerl_b200.parallel.cp import merge_zigzag
    want_logits, _ = _single()
    got = run_world(2, _cp_rank, False)
    logits = merge_zigzag([torch.from_numpy(g[0]) for g in got]).numpy()
    assert _rel(logits, want_logits) > 1e-3


def test_zigzag_roundtrip_and_balance():
    from tilerl_b200.parallel.cp import chunk_order, merge_zigzag, split_zigzag
    x = torch.arange(2 * 48).view(2, 48)
    parts = [split_zigzag(x, 4, r) for r in range(4)]
    assert torch.equal(merge_zigzag(parts), x)
    # causal work (sum of positions) is equal across ranks
    work = [int(p[0].sum()) for p in parts]
    assert len(set(work)) == 1
    assert chunk_order(2) == [(0, 0), (1, 0), (1, 1), (0, 1)]
