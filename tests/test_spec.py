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
