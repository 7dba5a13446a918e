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
