"""ZeRO-3 and plain data-parallel gates on CPU ranks (gloo): a sharded step on W ranks, each
with its own micro-batch, must equal one full-batch AdamW step on a single rank; sharded
checkpoints must resume exactly; each gate has a mutation that must fail."""
import pytest
import torch

from world_helpers import run_world


def _model(seed=3):
    from tilerl_b200.config import tiny_hybrid
    from tilerl_b200.models.hybrid import HybridModel
    cfg = tiny_hybrid()
    return cfg, HybridModel.build_random(cfg, seed=seed, keep_master=True)


def _data(cfg, world):
    g = torch.Generator().manual_seed(9)
    return torch.randint(0, cfg.vocab, (2 * world, 12), generator=g)


def _snapshot(model):
    # numpy arrays pickle by value (tensors would travel as shared-memory handles of a child that exits)
    return {k: v.detach().float().numpy().copy() for k, v in model.trainable("full").items()}


def _single_step(world, steps=2):
    from tilerl_b200 import rl
    from tilerl_b200.optim import AdamW
    cfg, model = _model()
    ids = _data(cfg, world)
    opt = AdamW(model.trainable("full"), lr=1e-3)
    for _ in range(steps):
        rl.train_step(model, ids, opt, max_norm=1.0)
    return _snapshot(model)


def _zero3_rank(rank, world, bug, steps, ckpt_dir):
    import torch.distributed as dist
    from tilerl_b200 import rl
    from tilerl_b200.parallel.zero3 import Zero3
    cfg, model = _model()
    ids = _data(cfg, world)[2 * rank:2 * rank + 2]
    comm = None
    if bug:
        from tilerl_b200.parallel.zero3 import TorchComm

        class LocalOnly(TorchComm):   # mutation: the gradient of the other ranks never arrives
            def reduce_scatter(self, full, shard_out, scale, accumulate):
                n = shard_out.numel()
                red = full.float()[self.rank * n:(self.rank + 1) * n]
                shard_out.add_(red) if accumulate else shard_out.copy_(red)
        comm = LocalOnly(dist.group.WORLD)
    z = Zero3(model, dist.group.WORLD, lr=1e-3, max_norm=1.0, comm=comm)
    full_bytes = sum(u.numel for u in z.units) * 16
    assert z.shard_bytes() <= full_bytes / world + 64 * len(z.units) * world
    for s in range(steps):
        if ckpt_dir and s == 1:
            torch.save(z.state_dict(), f"{ckpt_dir}/zero_{rank}.pt")
            cfg2, model2 = _model()
            with torch.no_grad():                   # wrong trainable weights: the shard must win
                for p in model2.trainable("full").values():
                    p.mul_(0.5)
            z = Zero3(model2, dist.group.WORLD, lr=1e-3, max_norm=1.0)
            z.load_state_dict(torch.load(f"{ckpt_dir}/zero_{rank}.pt", weights_only=False))
            model = model2
        rl.train_step(model, ids, z, max_norm=0.0, checkpoint_layers=True, on_grad=z.on_grad, hook=z)
    assert all(p.numel() == 0 for n, p in z.params.items() if n.startswith("master.L")), "layers not dropped"
    z.gather_all()
    out = _snapshot(model)
    return out, dict(z.stats)


def _dp_rank(rank, world):
    """Replicated parameters, gradients averaged with one all-reduce per tensor."""
    import torch.distributed as dist
    from tilerl_b200 import rl
    from tilerl_b200.optim import AdamW, clip_grad_norm
    cfg, model = _model()
    ids = _data(cfg, world)[2 * rank:2 * rank + 2]
    opt = AdamW(model.trainable("full"), lr=1e-3)
    for _ in range(2):
        st = rl.policy_step  # noqa: F841  (same step path as train_step below)
        b, t = ids.shape
        targets = torch.roll(ids, -1, 1)
        mask = (torch.arange(t)[None, :] < t - 1).float().expand(b, t) / (b * (t - 1))
        _, grads, _ = rl.forward_backward(model, ids, targets, lambda lg: mask, trainable=model.trainable("full"))
        for k in sorted(grads):
            dist.all_reduce(grads[k])
            grads[k] /= world
        clip_grad_norm(grads, 1.0)
        opt.step(grads)
    return _snapshot(model)


def _update_error(a, b):
    """Relative L2 distance between the two *updates* (parameters minus the common start):
    Adam normalises every element, so an element-wise tolerance would hinge on gradients
    that are zero up to rounding."""
    init = _snapshot(_model()[1])
    num = den = 0.0
    for k in b:
        da, db = torch.from_numpy(a[k] - init[k]).double(), torch.from_numpy(b[k] - init[k]).double()
        num += float((da - db).pow(2).sum())
        den += float(db.pow(2).sum())
    return (num / den) ** 0.5


def _close(a, b, tol=1e-3):
    return _update_error(a, b) < tol


@pytest.mark.parametrize("world", [2, 4])
def test_zero3_equals_single_rank_full_batch(world):
    got = run_world(world, _zero3_rank, False, 2, None)
    want = _single_step(world)
    for snap, stats in got:
        assert _close(snap, want)
        assert stats["reduce_scatters"] >= 2 * 3 and stats["gathers"] >= stats["reduce_scatters"]


def test_zero3_negative_control_no_reduction():
    got = run_world(2, _zero3_rank, True, 2, None)
    assert _update_error(got[0][0], _single_step(2)) > 0.05


def test_zero3_sharded_checkpoint_resumes_exactly(tmp_path):
    got = run_world(2, _zero3_rank, False, 2, str(tmp_path))
    want = _single_step(2)
    assert _close(got[0][0], want) and _close(got[1][0], want)


def test_dp_allreduce_equals_single_rank():
    got = run_world(4, _dp_rank)
    want = _single_step(4)
    assert all(_close(g, want) for g in got)


def test_zero3_world1_matches_adamw():
    from tilerl_b200 import rl
    from tilerl_b200.parallel.zero3 import Zero3
    cfg, model = _model()
    ids = _data(cfg, 1)
    z = Zero3(model, None, lr=1e-3, max_norm=1.0)
    for _ in range(2):
        rl.train_step(model, ids, z, max_norm=0.0, checkpoint_layers=True, on_grad=z.on_grad, hook=z)
    z.gather_all()
    assert _close(_snapshot(model), _single_step(1))


def test_zero3_low_precision_working_copy_keeps_every_leaf_watched():
    """With a bf16 working copy the vector parameters (norms, GDN vectors) change dtype when they
    are dropped and re-gathered; every one of them must still be trained: no unit may reach the
    optimizer step with leaves that never received a gradient, and a norm weight must move."""
    from tilerl_b200 import rl
    from tilerl_b200.parallel.zero3 import Zero3
    cfg, model = _model()
    ids = _data(cfg, 1)
    z = Zero3(model, None, lr=1e-2, max_norm=0.0, work_dtype=torch.bfloat16)
    z.gather_all()
    before = {k: v.float().clone() for k, v in z.params.items() if k.endswith("norm1") or k.endswith("a_log")}
    assert before
    for _ in range(2):
        rl.train_step(model, ids, z, max_norm=0.0, checkpoint_layers=True, on_grad=z.on_grad, hook=z)
    assert z.stats.get("flushed", 0) == 0
    assert z.stats["reduce_scatters"] == 2 * sum(1 for u in z.units if u.names)
    z.gather_all()
    for k, v in before.items():
        assert not torch.equal(z.params[k].float(), v), k


def _resync_rank(rank, world):
    """ZeRO-3 over `world` ranks trains; the same ranks serve a TP=`world` NVFP4 model.  After a
    step + resync, every rank's shard must equal what quantising the updated full master and
    cutting it for that rank gives."""
    import torch.distributed as dist
    from tilerl_b200 import rl
    from tilerl_b200.formats import quantize_nvfp4
    from tilerl_b200.models.hybrid import HybridModel, linear_names
    from tilerl_b200.parallel.mesh import shard_param
    from tilerl_b200.parallel.resync import resync
    from tilerl_b200.parallel.zero3 import Zero3
    cfg, trainer = _model()
    rollout = HybridModel.build_random(cfg, seed=3, tp_rank=rank, tp=world)
    addr = {k: (v.wq.data_ptr() if hasattr(v, "wq") else v.data_ptr()) for k, v in rollout.params.items()}
    ids = _data(cfg, world)[2 * rank:2 * rank + 2]
    z = Zero3(trainer, dist.group.WORLD, lr=1e-2, max_norm=1.0)
    rl.train_step(trainer, ids, z, max_norm=0.0, checkpoint_layers=True, on_grad=z.on_grad, hook=z)
    before = rollout.params["L0.gate_up"].wq.clone()
    out = resync(z, rollout)
    assert out["bytes"] > 0 and rollout.weights_version == 1
    assert not torch.equal(before, rollout.params["L0.gate_up"].wq), "rollout weights did not change"
    assert addr == {k: (v.wq.data_ptr() if hasattr(v, "wq") else v.data_ptr()) for k, v in rollout.params.items()}
    z.gather_all()
    bad = []
    for name in linear_names(cfg):
        want = shard_param(cfg, name, quantize_nvfp4(trainer.params["master." + name].float()), rank, world)
        got = rollout.params[name]
        if not (torch.equal(got.wq, want.wq) and torch.equal(got.scale.view(torch.uint8), want.scale.view(torch.uint8))
                and torch.equal(got.tscale, want.tscale)):
            bad.append(name)
    norm_ok = torch.equal(rollout.params["L0.norm1"], trainer.params["L0.norm1"].float())
    return bad, norm_ok


def test_resync_writes_tp_shards_of_the_full_quantisation():
    for bad, norm_ok in run_world(2, _resync_rank):
        assert bad == [] and norm_ok
