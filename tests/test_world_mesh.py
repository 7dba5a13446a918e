"""Mesh gate on CPU ranks (gloo): world 4 = data parallel 2 x tensor parallel 2.  Every rank holds
its TP shard of the master weights and its DP slice of the batch; after the TP collectives inside
the tape (fork / all-reduce / vocab-parallel cross-entropy) and a DP mean of the gradients, each
rank must hold exactly its shard of the single-rank full-batch gradient."""
import pytest
import torch

from world_helpers import run_world


def _setup():
    from tilerl_b200.config import tiny_hybrid
    cfg = tiny_hybrid()
    g = torch.Generator().manual_seed(4)
    ids = torch.randint(0, cfg.vocab, (4, 10), generator=g)
    return cfg, ids


def _mask(b, t):
    return (torch.arange(t)[None, :] < t - 1).float().expand(b, t) / (b * (t - 1))


def _single():
    from tilerl_b200 import rl
    from tilerl_b200.models.hybrid import HybridModel
    cfg, ids = _setup()
    model = HybridModel.build_random(cfg, seed=6, keep_master=True)
    tr = model.trainable("full")
    m = _mask(*ids.shape)
    _, grads, _ = rl.forward_backward(model, ids, torch.roll(ids, -1, 1), lambda lg: m, trainable=tr)
    return {k: v.numpy().copy() for k, v in grads.items()}


def _mesh_rank(rank, world, skip_dp):
    import torch.distributed as dist
    from tilerl_b200 import rl
    from tilerl_b200.models.hybrid import HybridModel
    from tilerl_b200.parallel.mesh import Mesh
    cfg, ids = _setup()
    mesh = Mesh(dp=2, tp=2)
    dp_i, tp_i, _ = mesh.coords(rank)
    groups = {}
    for axis, gl in (("tp", mesh.tp_groups()), ("dp", mesh.dp_groups())):       # same order on every rank
        for members in gl:
            g = dist.new_group(members)
            if rank in members:
                groups[axis] = g
    model = HybridModel.build_random(cfg, seed=6, tp_rank=tp_i, tp=2, keep_master=True)
    tr = model.trainable("full")
    mine = ids[2 * dp_i:2 * dp_i + 2]
    m = _mask(*mine.shape)
    _, grads, lp = rl.forward_backward(model, mine, torch.roll(mine, -1, 1), None, trainable=tr,
                                       tp_group=groups["tp"], tp_world=2, lp_weights_fn=lambda lp_: m)
    out = {}
    for k in sorted(grads):
        g = grads[k].contiguous()
        if not skip_dp:
            dist.all_reduce(g, group=groups["dp"])
            g = g / 2
        out[k] = g.numpy().copy()
    return tp_i, out


def _check(got, want, cfg):
    from tilerl_b200.parallel.mesh import shard_param
    worst = 0.0
    for tp_i, grads in got:
        for k, g in grads.items():
            base = k[len("master."):] if k.startswith("master.") else k
            ref = shard_param(cfg, base, torch.from_numpy(want[k]), tp_i, 2)
            num = float((torch.from_numpy(g).double() - ref.double()).norm())
            den = float(ref.double().norm()) + 1e-12
            worst = max(worst, num / den)
    return worst


def test_mesh_dp2_tp2_gradients_equal_single_rank():
    cfg, _ = _setup()
    got = run_world(4, _mesh_rank, False)
    assert _check(got, _single(), cfg) < 2e-4


def test_mesh_negative_control_without_dp_mean():
    cfg, _ = _setup()
    got = run_world(4, _mesh_rank, True)
    assert _check(got, _single(), cfg) > 1e-2
