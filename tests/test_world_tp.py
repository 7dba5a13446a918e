"""Distributed gates on CPU ranks (gloo): tensor-parallel serving and training must equal
the single-rank result, and each gate has a mutation that must fail."""
import pytest
import torch

from world_helpers import run_world


def _tp_serve(rank, world, no_collective):
    import torch.distributed as dist
    from helpers import rand_prompts
    from tilerl_b200.config import tiny_hybrid
    from tilerl_b200.engine import Engine, SamplingParams
    from tilerl_b200.kv import GdnStatePool, PagedKvPool
    from tilerl_b200.models.hybrid import HybridModel
    from tilerl_b200.ops.backend import RefOps, TPContext
    cfg = tiny_hybrid()
    model = HybridModel.build_random(cfg, seed=1, tp_rank=rank, tp=world)
    ops = RefOps(TPContext(rank, 1 if no_collective else world, dist.group.WORLD))
    d = model.dims
    kv = PagedKvPool(cfg, 64, dtype=torch.float32, n_kv_heads=d.n_kv)
    st = GdnStatePool(cfg, 6, ring_dtype=torch.float32, n_v_heads=d.gdn_nv, n_k_heads=d.gdn_nk)
    eng = Engine(model, ops, kv, st)
    prompts = rand_prompts(cfg, 2, 24)
    return [r.tokens for r in eng.generate(prompts, SamplingParams(max_tokens=8))]


def _single():
    from helpers import make_engine, rand_prompts
    from tilerl_b200.config import tiny_hybrid
    from tilerl_b200.engine import SamplingParams
    cfg = tiny_hybrid()
    eng = make_engine(cfg)
    return [r.tokens for r in eng.generate(rand_prompts(cfg, 2, 24), SamplingParams(max_tokens=8))]


@pytest.mark.parametrize("world", [2, 4])
def test_tp_serving_equals_single_rank(world):
    got = run_world(world, _tp_serve, False)
    want = _single()
    assert all(g == want for g in got)


def test_tp_serving_negative_control_no_collective():
    got = run_world(2, _tp_serve, True)
    assert got[0] != _single()


# ---- training: one clipped optimizer step under TP equals the single-rank step -------------------
def _train_setup():
    from tilerl_b200.config import tiny_hybrid
    cfg = tiny_hybrid()
    g = torch.Generator().manual_seed(8)
    return cfg, torch.randint(0, cfg.vocab, (2, 10), generator=g)


def _train_single(max_norm):
    from tilerl_b200 import rl
    from tilerl_b200.models.hybrid import HybridModel
    from tilerl_b200.optim import AdamW
    cfg, ids = _train_setup()
    model = HybridModel.build_random(cfg, seed=6, keep_master=True)
    tr = model.trainable("full")
    m = rl.train_step(model, ids, AdamW(tr, lr=1e-2), max_norm=max_norm)
    return m["grad_norm"], {k: v.detach().clone() for k, v in tr.items()}


def _train_rank(rank, world, max_norm, local_clip):
    import torch.distributed as dist
    from tilerl_b200 import rl
    from tilerl_b200.models.hybrid import HybridModel
    from tilerl_b200.optim import AdamW
    cfg, ids = _train_setup()
    model = HybridModel.build_random(cfg, seed=6, tp_rank=rank, tp=world, keep_master=True)
    tr = model.trainable("full")
    kw = dict(tp_group=dist.group.WORLD, tp_world=world)
    if local_clip:     # mutation: each rank clips by the norm of what it holds
        orig = rl._clip
        rl._clip = lambda grads, mn, fb: orig(grads, mn, {})
    m = rl.train_step(model, ids, AdamW(tr, lr=1e-2), max_norm=max_norm, **kw)
    return m["grad_norm"], {k: v.detach().numpy().copy() for k, v in tr.items()}


def _compare(got, want, cfg, world):
    from tilerl_b200.parallel.mesh import grad_is_sharded, shard_param
    worst_rep, worst = 0.0, 0.0
    for rank, (_, params) in enumerate(got):
        for k, v in params.items():
            base = k[len("master."):] if k.startswith("master.") else k
            v = torch.from_numpy(v)
            ref = shard_param(cfg, base, want[k], rank, world)
            err = float((v.double() - ref.double()).norm() / (ref.double().norm() + 1e-12))
            worst = max(worst, err)
            if not grad_is_sharded(k):
                worst_rep = max(worst_rep, float((v.double() - torch.from_numpy(got[0][1][k]).double()).abs().max()))
    return worst, worst_rep


def test_tp_train_step_clips_with_one_global_norm_and_matches_single_rank():
    """The gradient norm here is ~10x the clip threshold, so the coefficient matters: every TP rank
    must use the norm of the WHOLE gradient (sharded squares summed over ranks, replicated ones
    counted once), take the same step as one rank would, and keep replicated parameters identical."""
    cfg, _ = _train_setup()
    norm1, want = _train_single(0.05)
    got = run_world(2, _train_rank, 0.05, False)
    assert norm1 > 0.2                                     # the clip is active
    for n, _ in got:
        assert abs(n - norm1) < 2e-3 * norm1
    worst, worst_rep = _compare(got, want, cfg, 2)
    assert worst < 2e-3 and worst_rep < 1e-6


def test_tp_train_step_negative_control_local_norm():
    cfg, _ = _train_setup()
    norm1, want = _train_single(0.05)
    got = run_world(2, _train_rank, 0.05, True)
    assert any(abs(n - norm1) > 1e-2 * norm1 for n, _ in got)
