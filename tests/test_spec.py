"""Speculative decoding: outputs are identical with and without a drafter (greedy and seeded
sampling), acceptance bookkeeping, GDN state rollback through the per-token state planes."""
import torch

from helpers import make_engine, rand_prompts
from tilerl_b200.config import tiny_hybrid
from tilerl_b200.engine import SamplingParams
from tilerl_b200.spec import (BlockDrafter, ChainDrafter, ConstantDrafter, OracleDrafter, expected_goodput,
                              verify_lens)


def _run(cfg, prompts, sp, drafter=None, width=0, model=None):
    eng = make_engine(cfg, model=model, drafter=drafter, spec_width=width, planes=max(1, width), blocks=160)
    return [r.tokens for r in eng.generate(prompts, sp)], eng


def test_verify_lens_and_goodput():
    assert verify_lens([1, 2, 3], [1, 2, 9]) == 2 and verify_lens([], [5]) == 0
    assert abs(expected_goodput(1.0, 8) - 8) < 1e-9 and expected_goodput(0.0, 8) == 1.0


def test_spec_on_equals_spec_off_for_every_drafter():
    cfg = tiny_hybrid()
    prompts = rand_prompts(cfg, 2, 20, seed=4)
    for sp in (SamplingParams(max_tokens=14), SamplingParams(max_tokens=10, temperature=1.0, top_p=0.9, seed=7)):
        want, base = _run(cfg, prompts, sp)
        model = base.model
        cont = {tuple(p): w for p, w in zip(prompts, want)}
        for name, d, w in (("block", BlockDrafter(model), 4), ("chain", ChainDrafter(model), 4),
                           ("oracle", OracleDrafter(cont), 8), ("const", ConstantDrafter(3), 8)):
            got, eng = _run(cfg, prompts, sp, drafter=d, width=w, model=model)
            assert got == want, name
            c = eng.counters
            assert c["spec_drafted"] > 0
            if name == "oracle":
                assert c["spec_accepted"] == c["spec_drafted"]          # forced full acceptance
                assert c["decode_ticks"] + c["mixed_ticks"] < len(want[0])  # several tokens per tick
            if name == "const":
                assert c["spec_accepted"] <= 2
            assert eng.kv.used_blocks == 0


def test_spec_with_chunked_prefill_and_prefix_cache():
    from tilerl_b200.engine import StepLimits
    from tilerl_b200.kv import PrefixStore
    cfg = tiny_hybrid()
    prompts = rand_prompts(cfg, 2, 40, seed=9)
    sp = SamplingParams(max_tokens=9)
    want, base = _run(cfg, prompts, sp)
    cont = {tuple(p): w for p, w in zip(prompts, want)}
    eng = make_engine(cfg, model=base.model, drafter=OracleDrafter(cont), spec_width=4, planes=4, blocks=200,
                      limits=StepLimits(max_batched_tokens=16, prefill_align=8))
    eng.prefix = PrefixStore(eng.kv)
    assert [r.tokens for r in eng.generate(prompts, sp)] == want
    assert [r.tokens for r in eng.generate(prompts, sp)] == want     # second pass: prefix hits
    assert eng.prefix.hits == 2


def test_drafter_checkpoint_round_trip(tmp_path):
    """A saved drafter loads back with identical tensors and proposes the same drafts, so serving
    with it gives the same counters; a drafter for another trunk width is refused."""
    import pytest
    from tilerl_b200.config import tiny
    from tilerl_b200.models.hybrid import HybridModel
    from tilerl_b200.spec import BlockDrafterConfig, load_drafter, save_drafter
    cfg = tiny_hybrid()
    prompts = rand_prompts(cfg, 2, 20, seed=4)
    sp = SamplingParams(max_tokens=12)
    want, base = _run(cfg, prompts, sp)
    model = base.model
    for name, d in (("block", BlockDrafter(model, BlockDrafterConfig(width=4, n_layers=1), seed=5)),
                    ("chain", ChainDrafter(model, seed=5))):
        path = str(tmp_path / name)
        save_drafter(d, path)
        d2 = load_drafter(model, path)
        assert type(d2) is type(d) and d2.aux_layers == d.aux_layers
        if name == "block":
            assert all(torch.equal(d.p[k], d2.p[k]) for k in d.p)
        got1, e1 = _run(cfg, prompts, sp, drafter=d, width=4, model=model)
        got2, e2 = _run(cfg, prompts, sp, drafter=d2, width=4, model=model)
        assert got1 == got2 == want
        assert e1.counters["spec_accepted"] == e2.counters["spec_accepted"]
    other = HybridModel.build_random(tiny(), seed=0)
    if other.cfg.hidden != cfg.hidden:
        with pytest.raises(ValueError):
            load_drafter(other, str(tmp_path / "block"))


def _drafter(width=4, **kw):
    from tilerl_b200.models.hybrid import HybridModel
    from tilerl_b200.spec import BlockDrafterConfig
    cfg = tiny_hybrid()
    model = HybridModel.build_random(cfg, seed=0)
    return cfg, BlockDrafter(model, BlockDrafterConfig(width=width, n_layers=2, n_heads=4, n_kv_heads=2, **kw), seed=3)


def test_block_drafter_conv_is_identity_at_init_and_zero_padded_at_the_block_start():
    """The grouped two-tap conv along the block: with the initial coefficients it passes its input
    through; with a second tap, slot j reads slot j - 1 only, and slot 0 reads nothing before it."""
    cfg, d = _drafter()
    w, h = d.cfg.width, cfg.hidden
    g = torch.Generator().manual_seed(0)
    x = torch.randn(w, h, generator=g)
    zero = torch.zeros(w, d.cfg.conv_taps, d.groups)
    base = d.p["l0.attn_conv.base"][0]
    assert torch.allclose(d._conv(x, zero, base), x)
    base2 = base.clone()
    base2[1] = 0.5                                           # tap 1: half of the slot before
    y = d._conv(x, zero, base2)
    assert torch.allclose(y[0], x[0]) and torch.allclose(y[1:], x[1:] + 0.5 * x[:-1], atol=1e-6)
    x2 = x.clone()
    x2[1] += 1.0                                             # a change in slot 1 reaches slots 1 and 2 only
    changed = (d._conv(x2, zero, base2) - y).abs().sum(-1) > 0
    assert changed.tolist() == [False, True, True, False]
    # per-slot offsets act on one group of channels
    delta = zero.clone()
    delta[2, 0, 1] = 1.0                                     # slot 2, tap 0, group 1: coefficient 2 instead of 1
    z = d._conv(x, delta, base)
    gs = d.gsize
    assert torch.allclose(z[2, gs:2 * gs], 2 * x[2, gs:2 * gs]) and torch.allclose(z[2, :gs], x[2, :gs])
    assert torch.allclose(z[[0, 1, 3]], x[[0, 1, 3]])


def test_block_drafter_selector_walk_is_argmax_until_trained_and_then_follows_the_pairwise_term():
    cfg, d = _drafter(top_k=4, sel_rank=4)
    g = torch.Generator().manual_seed(1)
    hid = torch.randn(3, cfg.hidden, generator=g)
    plain = d._head(hid).argmax(-1).tolist()
    assert d.paths(hid, anchor=5) == plain                   # succ == 0: the pairwise term vanishes
    # make the runner-up of slot 1 the strongly preferred successor of the token chosen for slot 0
    logits = d._head(hid)
    top = torch.topk(logits, 4, dim=-1)
    runner_up, prev = int(top.indices[1, 1]), plain[0]
    proj1 = (hid[1] @ d.p["sel.proj"].t()).float()
    direction = d.p["sel.pred"][prev].float() * proj1
    d.p["sel.succ"][runner_up] = direction * (10.0 * float(top.values[1, 0] - top.values[1, 1] + 1.0) / float(direction.dot(direction)))
    walked = d.paths(hid, anchor=5)
    assert walked[0] == plain[0] and walked[1] == runner_up
    # the walk is sequential: another anchor only matters through slot 0's pairwise term
    assert d.paths(hid, anchor=6)[0] == plain[0]


def test_block_drafter_context_kv_grows_by_the_new_rows_and_matches_a_fresh_projection():
    """The per-request context K / V cache: rows are projected when they enter and appended; proposing
    from the cache gives the drafts of a drafter that projects the whole window again."""
    from types import SimpleNamespace
    cfg, d = _drafter()
    g = torch.Generator().manual_seed(2)
    eng = SimpleNamespace(spec_width=4)
    taps_all = {l: torch.randn(12, cfg.hidden, generator=g) for l in d.aux_layers}
    req = SimpleNamespace(rid=1, state="prefill", toks=[3, 4, 5], n_last_commit=1)
    first = d.propose(eng, req, {l: t[:8] for l, t in taps_all.items()}, 0, 8, 3)
    assert d.ctx_kv[1][0].shape[0] == 8
    req.state, req.toks = "decode", [3, 4, 5, 6]
    second = d.propose(eng, req, {l: t[8:12] for l, t in taps_all.items()}, 0, 4, 3)   # 4 rows ran, 1 was committed
    assert d.ctx_kv[1][0].shape[0] == 9 and d.ctx[1].shape[0] == 9
    # from scratch: the same 9 context rows projected in one go
    _, d2 = _drafter()
    rows = {l: torch.cat([t[:8], t[8:9]]) for l, t in taps_all.items()}
    req2 = SimpleNamespace(rid=7, state="prefill", toks=[3, 4, 5, 6], n_last_commit=1)
    assert d2.propose(eng, req2, rows, 0, 9, 3) == second
    for a, b in zip(d.ctx_kv[1], d2.ctx_kv[7]):
        assert torch.allclose(a, b, atol=1e-6)
    assert len(first) == 3 and len(second) == 3
    d.release(1)
    assert 1 not in d.ctx_kv and 1 not in d.ctx
    # the window: a context longer than the window keeps its newest rows
    _, d3 = _drafter(window=6)
    d3.propose(eng, SimpleNamespace(rid=2, state="prefill", toks=[1], n_last_commit=1), taps_all, 0, 12, 2)
    assert d3.ctx_kv[2][0].shape[0] == 6


class _FakeVerifyGraph:
    """Stands where the CUDA-graph verify runner stands, on the CPU: runs the same forward eagerly,
    walks every chain under greedy acceptance and selects the state plane -- what the graph's last
    kernel does on the device -- and hands the counts to the engine."""

    def __init__(self, eng):
        self.eng, self.replays = eng, 0

    def run(self, seqs, need_logits):
        from tilerl_b200.batch import Batch
        from tilerl_b200.graph import VerifyOut
        e = self.eng
        keep = max(len(s["tokens"]) for s in seqs)
        batch = Batch.build(seqs, e.device, keep_steps=keep)
        aux = tuple(e.drafter.aux_layers) if e.drafter is not None else ()
        res = e.model.forward(batch, e.ops, e.kv, e.states, last_only=False, aux_layers=aux)
        logits, taps = (res[0], res[2]) if aux else (res, None)
        amax = [int(t) for t in logits.argmax(-1).tolist()]
        accept, off = [], 0
        for s in seqs:
            chain, ok = s["tokens"], 0
            while ok + 1 < len(chain) and amax[off + ok] == chain[ok + 1]:
                ok += 1
            e.states.select_step(s["slot"], ok)
            accept.append(ok)
            off += len(chain)
        self.replays += 1
        return VerifyOut(logits, amax, taps, accept)


def test_engine_commits_from_device_side_accept_counts_like_the_host_walk():
    """With accept counts handed over by the verify runner the engine only commits: same tokens and
    acceptance counters as its own host walk, for a drafter that is always right, one that never is,
    and the block drafter; sampling requests keep the host walk."""
    cfg = tiny_hybrid()
    prompts = rand_prompts(cfg, 2, 20, seed=4)
    sp = SamplingParams(max_tokens=14)
    want, base = _run(cfg, prompts, sp)
    model = base.model
    cont = {tuple(p): w for p, w in zip(prompts, want)}
    for name, mk in (("oracle", lambda: OracleDrafter(cont)), ("const", lambda: ConstantDrafter(3)),
                     ("block", lambda: BlockDrafter(model, seed=1))):
        host_tokens, host = _run(cfg, prompts, sp, drafter=mk(), width=4, model=model)
        eng = make_engine(cfg, model=model, drafter=mk(), spec_width=4, planes=4, blocks=160)
        eng.vgraph = _FakeVerifyGraph(eng)
        got = [r.tokens for r in eng.generate(prompts, sp)]
        assert got == host_tokens == want, name
        assert eng.vgraph.replays > 0 and eng.counters["spec_device_accepts"] > 0, name
        assert (eng.counters["spec_drafted"], eng.counters["spec_accepted"]) == \
            (host.counters["spec_drafted"], host.counters["spec_accepted"]), name
        assert host.counters["spec_device_accepts"] == 0
    # a request that samples: the runner's counts are ignored, the host walk decides
    sps = SamplingParams(max_tokens=10, temperature=1.0, top_p=0.9, seed=7)
    want_s, _ = _run(cfg, prompts, sps, model=model)
    eng = make_engine(cfg, model=model, drafter=OracleDrafter({tuple(p): w for p, w in zip(prompts, want_s)}),
                      spec_width=4, planes=4, blocks=160)
    eng.vgraph = _FakeVerifyGraph(eng)
    assert [r.tokens for r in eng.generate(prompts, sps)] == want_s
    assert eng.counters["spec_device_accepts"] == 0
