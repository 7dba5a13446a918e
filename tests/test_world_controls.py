"""Mutation controls of the distributed gates (CPU ranks over gloo).

A gate that compares a multi-rank run with the single-rank run proves something only if breaking
the distributed part makes it fail.  Every case here runs one gate with one collective, halo, fold
or shard rule broken inside the worker process (the product code is patched in that process only)
and asserts that the gate's own metric moves past its pass threshold.  The table at the end keeps
the list honest: every world gate file has at least one control.

Parity: the reference's table of 23 controls over 14 gates
(tests/test_world_negative_controls.py:81-105).
"""
import glob
import os

import torch

import test_world_cp as gate_cp
import test_world_mesh as gate_mesh
import test_world_tp as gate_tp
import test_world_zero3 as gate_z
from world_helpers import run_world


# ---- context parallelism ---------------------------------------------------------------------------
def _cp_mutated(rank, world, mutation):
    from tilerl_b200.parallel import cp as CP
    if mutation == "no-compose":          # every chunk starts from a zero GDN state
        CP.fold_entry_states = lambda a, b, cp: torch.zeros_like(b)
    elif mutation == "decay-identity":    # the fold forgets the decay: S <- S + B_j
        fold = CP.fold_entry_states
        eye = lambda a: torch.eye(a.shape[-1], dtype=a.dtype).expand_as(a).contiguous()   # noqa: E731
        CP.fold_entry_states = lambda a, b, cp: fold(eye(a), b, cp)
    elif mutation == "slice-bwd":         # all-gather backward keeps the local slice, no sum over ranks
        def bwd(ctx, g):
            return g[ctx.cp.rank].contiguous(), None
        CP._AllGather.backward = staticmethod(bwd)
    elif mutation == "local-positions":   # causal mask and RoPE from rank-local positions
        CP.positions_for = lambda seq_len, cp: torch.arange(seq_len // cp.world)
        gate_cp.__dict__["_patched_positions"] = True
    elif mutation == "kv-not-gathered":   # no exchange: every slot of the gathered K / V holds this rank's own rows
        gather0 = CP.gather_kv

        def own_only(k, v, pos, cp):
            _, _, pa = gather0(k, v, pos, cp)
            return torch.cat([k] * cp.world, 1), torch.cat([v] * cp.world, 1), pa
        CP.gather_kv = own_only
    elif mutation == "kv-positions-local":  # the gathered keys all carry this rank's positions: the causal mask is wrong
        gather = CP.gather_kv

        def gather_kv(k, v, pos, cp):
            ka, va, _ = gather(k, v, pos, cp)
            return ka, va, pos.repeat(cp.world)
        CP.gather_kv = gather_kv
    return gate_cp._cp_rank(rank, world, True)


def _cp_metrics(mutation):
    from tilerl_b200.parallel.cp import merge_zigzag
    want_logits, want_grads = gate_cp._single()
    got = run_world(2, _cp_mutated, mutation)
    logits = merge_zigzag([torch.from_numpy(g[0]) for g in got]).numpy()
    worst_grad = max(gate_cp._rel(got[0][1][n], g) for n, g in want_grads.items())
    return gate_cp._rel(logits, want_logits), worst_grad


def test_cp_control_gdn_states_not_composed_across_ranks():
    logits, _ = _cp_metrics("no-compose")
    assert logits > 1e-3


def test_cp_control_fold_without_decay():
    logits, _ = _cp_metrics("decay-identity")
    assert logits > 1e-3


def test_cp_control_all_gather_backward_keeps_local_slice():
    logits, grads = _cp_metrics("slice-bwd")
    assert logits < 1e-4          # the forward is untouched ...
    assert grads > 2e-2           # ... the gradients are not summed over the ranks that used the K / V rows


def test_cp_control_rank_local_positions():
    logits, _ = _cp_metrics("local-positions")
    assert logits > 1e-3


def test_cp_control_keys_of_other_ranks_never_gathered():
    logits, _ = _cp_metrics("kv-not-gathered")
    assert logits > 1e-3


def test_cp_control_gathered_keys_carry_local_positions():
    logits, _ = _cp_metrics("kv-positions-local")
    assert logits > 1e-3


# ---- tensor parallelism -----------------------------------------------------------------------------
def _tp_serve_mutated(rank, world, mutation):
    import torch.distributed as dist
    from helpers import rand_prompts
    from tilerl_b200.config import tiny_hybrid
    from tilerl_b200.engine import Engine, SamplingParams
    from tilerl_b200.kv import GdnStatePool, PagedKvPool
    from tilerl_b200.models.hybrid import HybridModel
    from tilerl_b200.ops.backend import RefOps, TPContext
    cfg = tiny_hybrid()
    shard_rank = 0 if mutation == "rank0-shard" else rank          # every rank loads rank 0's shard
    model = HybridModel.build_random(cfg, seed=1, tp_rank=shard_rank, tp=world)
    ops = RefOps(TPContext(rank, world, dist.group.WORLD))
    if mutation == "no-vocab-gather":                                # argmax over the local vocabulary shard only
        ops.all_gather_last = lambda x: x
    d = model.dims
    kv = PagedKvPool(cfg, 64, dtype=torch.float32, n_kv_heads=d.n_kv)
    st = GdnStatePool(cfg, 6, ring_dtype=torch.float32, n_v_heads=d.gdn_nv, n_k_heads=d.gdn_nk)
    eng = Engine(model, ops, kv, st)
    return [r.tokens for r in eng.generate(rand_prompts(cfg, 2, 24), SamplingParams(max_tokens=8))]


def test_tp_control_every_rank_loads_rank0_shard():
    got = run_world(2, _tp_serve_mutated, "rank0-shard")
    assert got[0] != gate_tp._single()


def test_tp_control_vocabulary_shards_not_gathered():
    got = run_world(2, _tp_serve_mutated, "no-vocab-gather")
    assert got[0] != gate_tp._single() or got[1] != gate_tp._single()


def _tp_train_mutated(rank, world, mutation):
    from tilerl_b200 import rl
    from tilerl_b200 import tape as T
    if mutation == "local-head-norm-grads":
        # q / k / GDN norm weights are replicated but see only this rank's heads: without the sum over
        # the TP group every rank keeps a partial gradient
        rl.tp_sync_replicated_grads = lambda grads, group: None
    elif mutation == "no-fork":
        # the identity-forward / all-reduce-backward at the entry of a column-parallel block is dropped
        T.tp_fork = lambda tape, x: x
    elif mutation == "ce-local-max":
        # the vocabulary-sharded cross entropy skips the max over ranks: every rank exponentiates against
        # its own maximum and the summed denominators do not belong together
        import torch.distributed as dist
        real = dist.all_reduce

        def all_reduce(t, op=dist.ReduceOp.SUM, group=None, **kw):
            return None if op == dist.ReduceOp.MAX else real(t, op=op, group=group, **kw)
        dist.all_reduce = all_reduce
    return gate_tp._train_rank(rank, world, 1e9, False)


def _tp_train_worst(mutation):
    cfg, _ = gate_tp._train_setup()
    _, want = gate_tp._train_single(1e9)
    got = run_world(2, _tp_train_mutated, mutation)
    return gate_tp._compare(got, want, cfg, 2)


def test_tp_train_control_without_mutation_matches():
    worst, worst_rep = _tp_train_worst("none")
    assert worst < 2e-3 and worst_rep < 1e-6


def test_tp_train_control_head_norm_gradients_not_summed():
    worst, worst_rep = _tp_train_worst("local-head-norm-grads")
    assert worst > 1e-2 or worst_rep > 1e-4


def test_tp_train_control_without_fork():
    worst, worst_rep = _tp_train_worst("no-fork")
    assert worst > 1e-2 or worst_rep > 1e-4


def test_tp_train_control_sharded_cross_entropy_with_rank_local_max():
    worst, worst_rep = _tp_train_worst("ce-local-max")
    assert worst > 1e-2 or worst_rep > 1e-4


# ---- mesh (dp x tp) ---------------------------------------------------------------------------------
def _mesh_mutated(rank, world, mutation):
    import torch.distributed as dist
    from tilerl_b200.parallel.mesh import Mesh
    if mutation == "ungrouped":
        # tensor-parallel collectives run over the whole world instead of the rank's TP group
        real = dist.new_group
        dist.new_group = lambda members=None, **kw: (dist.group.WORLD if len(members) == 2 and
                                                     members in Mesh(dp=2, tp=2).tp_groups() else real(members, **kw))
    elif mutation == "same-batch":
        # both data-parallel replicas read the first half of the batch
        gate_mesh.__dict__["_setup_orig"] = gate_mesh._setup

        def setup():
            cfg, ids = gate_mesh._setup_orig()
            return cfg, torch.cat([ids[:2], ids[:2]])
        gate_mesh._setup = setup
    elif mutation == "transposed-coords":
        # a rank reads its (dp, tp) coordinates with the axes swapped while the groups follow the real
        # formula: two members of one TP group hold the same shard
        Mesh.coords = lambda self, r: (r % self.dp, r // self.dp, 0)
    return gate_mesh._mesh_rank(rank, world, False)


def test_mesh_control_tp_collectives_over_the_whole_world():
    cfg, _ = gate_mesh._setup()
    got = run_world(4, _mesh_mutated, "ungrouped")
    assert gate_mesh._check(got, gate_mesh._single(), cfg) > 1e-2


def test_mesh_control_replicas_read_the_same_half_batch():
    cfg, _ = gate_mesh._setup()
    got = run_world(4, _mesh_mutated, "same-batch")
    assert gate_mesh._check(got, gate_mesh._single(), cfg) > 1e-2


def test_mesh_control_rank_coordinates_transposed():
    cfg, _ = gate_mesh._setup()
    got = run_world(4, _mesh_mutated, "transposed-coords")
    assert gate_mesh._check(got, gate_mesh._single(), cfg) > 1e-2


# ---- ZeRO-3 / data parallel -------------------------------------------------------------------------
def _zero3_mutated(rank, world, mutation):
    from tilerl_b200.parallel import zero3 as Z
    if mutation == "wrong-shard":
        # the reduce-scatter hands every rank its neighbour's slice of the summed gradient
        def reduce_scatter(self, full, shard_out, scale, accumulate):
            import torch.distributed as dist
            n = shard_out.numel()
            buf = full.float().clone()
            dist.all_reduce(buf, group=self.group)
            r = (self.rank + 1) % self.world
            red = buf[r * n:(r + 1) * n] * scale
            shard_out.add_(red) if accumulate else shard_out.copy_(red)
        Z.TorchComm.reduce_scatter = reduce_scatter
    elif mutation == "stale-gather":
        # the all-gather never talks: every slot of the full parameter is this rank's own shard
        def all_gather(self, shard, full, stream=None):
            full.view(self.world, -1).copy_(shard.to(full.dtype).view(1, -1).expand(self.world, -1))
        Z.TorchComm.all_gather = all_gather
    elif mutation == "rotated-gather":
        # the all-gather delivers every shard one slot too far: the full parameter is a rotation of itself
        def all_gather(self, shard, full, stream=None):
            import torch.distributed as dist
            parts = [torch.empty_like(shard) for _ in range(self.world)]
            dist.all_gather(parts, shard.contiguous(), group=self.group)
            full.view(self.world, -1).copy_(torch.stack(parts[1:] + parts[:1]).to(full.dtype))
        Z.TorchComm.all_gather = all_gather
    return gate_z._zero3_rank(rank, world, False, 2, None)


def test_zero3_control_reduce_scatter_returns_the_neighbours_slice():
    got = run_world(2, _zero3_mutated, "wrong-shard")
    assert gate_z._update_error(got[0][0], gate_z._single_step(2)) > 0.05


def test_zero3_control_all_gather_without_communication():
    got = run_world(2, _zero3_mutated, "stale-gather")
    assert gate_z._update_error(got[0][0], gate_z._single_step(2)) > 0.05


def test_zero3_control_all_gather_rotates_the_shards():
    got = run_world(2, _zero3_mutated, "rotated-gather")
    assert gate_z._update_error(got[0][0], gate_z._single_step(2)) > 0.05


def _dp_mutated(rank, world):
    import torch.distributed as dist
    dist.all_reduce = lambda t, *a, **k: None      # replicas never average their gradients
    return gate_z._dp_rank(rank, world)


def test_dp_control_without_gradient_all_reduce():
    got = run_world(2, _dp_mutated)
    assert gate_z._update_error(got[0], gate_z._single_step(2)) > 0.05 or \
        gate_z._update_error(got[0], got[1]) > 1e-3


# ---- the table ------------------------------------------------------------------------------------------
CONTROLS = {
    "test_world_cp.py": ["test_cp_negative_control_without_halo", "test_cp_control_gdn_states_not_composed_across_ranks",
                         "test_cp_control_fold_without_decay", "test_cp_control_all_gather_backward_keeps_local_slice",
                         "test_cp_control_rank_local_positions", "test_cp_control_keys_of_other_ranks_never_gathered",
                         "test_cp_control_gathered_keys_carry_local_positions"],
    "test_world_tp.py": ["test_tp_serving_negative_control_no_collective", "test_tp_train_step_negative_control_local_norm",
                         "test_tp_control_every_rank_loads_rank0_shard", "test_tp_control_vocabulary_shards_not_gathered",
                         "test_tp_train_control_head_norm_gradients_not_summed", "test_tp_train_control_without_fork",
                         "test_tp_train_control_sharded_cross_entropy_with_rank_local_max"],
    "test_world_mesh.py": ["test_mesh_negative_control_without_dp_mean", "test_mesh_control_tp_collectives_over_the_whole_world",
                           "test_mesh_control_replicas_read_the_same_half_batch",
                           "test_mesh_control_rank_coordinates_transposed"],
    "test_world_zero3.py": ["test_zero3_negative_control_no_reduction",
                            "test_zero3_control_reduce_scatter_returns_the_neighbours_slice",
                            "test_zero3_control_all_gather_without_communication", "test_dp_control_without_gradient_all_reduce",
                            "test_zero3_control_all_gather_rotates_the_shards"],
}


def test_every_world_gate_has_a_control_and_every_listed_control_exists():
    here = os.path.dirname(__file__)
    gates = {os.path.basename(p) for p in glob.glob(os.path.join(here, "test_world_*.py"))} - {"test_world_controls.py"}
    assert gates == set(CONTROLS), gates ^ set(CONTROLS)
    source = "".join(open(p).read() for p in glob.glob(os.path.join(here, "test_world_*.py")))
    for names in CONTROLS.values():
        for n in names:
            assert f"def {n}(" in source, n
    assert sum(len(v) for v in CONTROLS.values()) >= 23
