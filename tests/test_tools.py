"""Cost model, memory planner, ledger, bench store, recipes, merge, eval helpers, generate."""
import json
import os

import pytest
import torch

from tilerl_b200 import benchrec, evals, kernel_cost as kc, ledger, memory, merge, recipes
from tilerl_b200.calibration import load_peaks
from tilerl_b200.config import qwen38_27b, tiny_hybrid


def test_cost_model_matches_hand_arithmetic():
    cfg = qwen38_27b()
    rows = kc.tick_rows(cfg, kc.TickShape())
    by = {r.name: r for r in rows}
    gu = by["mlp.gate_up (norm + swiglu fused)"]
    assert gu.count == 64 and abs(gu.bytes - (34816 * 5120 * 0.5625 + 4 + 5120 * 2 + 34816 * 2)) < 1
    assert 15e9 < kc.tick_bytes(rows) < 18e9
    pk = load_peaks()
    b1 = kc.bound_seconds(rows, pk.hbm_gbs, pk.bf16_tflops)
    b8 = kc.bound_seconds(kc.tick_rows(cfg, kc.TickShape(tp=8)), pk.hbm_gbs, pk.bf16_tflops)
    assert 2e-3 < b1 < 3.5e-3 and b8 < b1 / 5
    assert "total" in kc.table(rows, pk.hbm_gbs, pk.bf16_tflops)
    assert kc.bound_seconds(kc.prefill_rows(cfg, 512), pk.hbm_gbs, pk.bf16_tflops) > 2e-3


def test_memory_plan_fits_and_reports():
    cfg = qwen38_27b()
    p = memory.plan(cfg)
    assert p.total < memory.B200_BYTES and p.blocks > 10000
    assert "kv pool" in memory.memory_table(p, peak=p.total + 5 * memory.GIB)
    full = memory.train_plan(cfg, mode="full", zero=8)
    assert sum(full.values()) < 100 * memory.GIB          # ZeRO-3 over 8 ranks fits
    assert sum(memory.train_plan(cfg, mode="full", zero=1).values()) > memory.B200_BYTES
    assert memory.plan(cfg, device_bytes=10 * memory.GIB).notes[0].startswith("model does not fit")


def test_ledger_and_early_stop(tmp_path):
    r = ledger.Run({"recipe": "x", "lr": 1e-5}, root=str(tmp_path))
    r2 = ledger.Run({"recipe": "x", "lr": 1e-5}, root=str(tmp_path))
    assert r.id == r2.id and len(r.id) == 12
    r.log(step=1, score=0.5), r.log(step=2, score=0.8)
    assert r.gate("score", 0.8, 0.7) and not r.gate("loss", 2.0, 1.0, higher_is_better=False)
    r.finish()
    man = ledger.load_run(r.id, str(tmp_path))
    assert man["status"] == "gate_failed" and ledger.time_to_score(man, "score", 0.75) is not None
    child = ledger.Run({"recipe": "y"}, root=str(tmp_path), parent=r.id)
    assert ledger.lineage(child.id, str(tmp_path)) == [child.id, r.id]
    es = ledger.EarlyStop(patience=2)
    assert [es.update(s, i) for i, s in enumerate([0.1, 0.3, 0.2, 0.25])] == [False, False, False, True]
    assert es.best_step == 1


def test_bench_store_schema_and_gate(tmp_path):
    path = str(tmp_path / "m.jsonl")
    shape = dict(model="27b", batch=1, ctx=512, tp=1)
    benchrec.append(benchrec.make_record("decode_tok_s", 130.0, shape, floor=400.0), path)
    recs = benchrec.load(path)
    assert recs[0]["status"] == "ok"
    assert benchrec.gate(benchrec.make_record("decode_tok_s", 128.0, shape), recs)["passed"]
    assert not benchrec.gate(benchrec.make_record("decode_tok_s", 100.0, shape), recs)["passed"]
    assert benchrec.validate(benchrec.make_record("decode_tok_s", 500.0, shape, floor=400.0))["status"] == "IMPLAUSIBLE"
    for bad in (dict(metric="nope"), dict(unit="ms"), dict(shape={}), dict(warm=1)):
        with pytest.raises(benchrec.SchemaError):
            benchrec.validate({**benchrec.make_record("decode_tok_s", 1.0, shape), **bad})
    assert len(benchrec.METRICS) >= 19


def test_recipes_and_merge_methods():
    assert recipes.expand("grpo-tiny-smoke", {"steps": 9, "lr": None})["steps"] == 9
    with pytest.raises(KeyError):
        recipes.expand("nope", {})
    torch.manual_seed(0)
    d = [torch.randn(8, 6), torch.randn(8, 6)]
    assert torch.allclose(merge.merge_average(d), (d[0] + d[1]) / 2)
    t = merge.merge_ties(d, density=0.5)
    assert t.shape == (8, 6) and (t != 0).sum() <= 48
    assert merge.merge_dare(d, drop=0.5).shape == (8, 6)
    iso = merge.merge_iso(d)
    sv = torch.linalg.svdvals(iso)
    assert torch.allclose(sv, sv.mean().expand_as(sv), atol=1e-4)


def test_answer_matching_rewards_and_judge():
    assert evals.last_boxed("so \\boxed{\\frac{1}{2}} ok") == "\\frac{1}{2}"
    assert evals.answers_match("\\frac{1}{2}", "0.5") and evals.answers_match("1,000", "1000")
    assert evals.gsm8k_answer("steps... #### 42") == "42" and evals.choice_answer("I pick (b). B") == "B"
    assert evals.reward_even([], [2, 4, 5, 7]) == 0.5 and evals.reward_mod7([], [1, 2, 3, 1]) == 1.0
    out = evals.judge_tiebreak([1.0, 1.0, 0.0], ["long answer", "x", "y"], lambda a, b: 1.0 if len(a) > len(b) else 0.0)
    assert out[0] > out[1] and out[2] == 0.0


def test_offline_generate_and_eval(tmp_path):
    from tilerl_b200.generate import generate, read_prompts
    pf = tmp_path / "p.jsonl"
    pf.write_text('{"prompt": "hello"}\nplain line\n\n{"prompt": "third"}\n')
    assert read_prompts(str(pf)) == ["hello", "plain line", "third"]
    files = generate("tiny", str(pf), str(tmp_path / "out"), workers=1, max_tokens=4)
    rows = [json.loads(l) for l in open(files[0])]
    assert len(rows) == 3 and all(r["tokens"] <= 4 for r in rows)
    from helpers import make_engine
    from tilerl_b200.tokenizer import ByteTokenizer
    from tilerl_b200.config import tiny
    eng = make_engine(tiny())
    res = evals.evaluate(eng, ByteTokenizer(), [{"question": "1+1?", "answer": "2"}], max_tokens=4)
    assert res["n"] == 1 and 0.0 <= res["accuracy"] <= 1.0


def test_committed_measurements_pass_the_schema_and_their_floors():
    """bench/measurements.jsonl (the measured figures of this build as records): every line
    validates, none beats its physical floor, and the headline shapes are present."""
    import os
    from tilerl_b200 import benchrec as B
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "bench", "measurements.jsonl")
    recs = B.load(path)
    assert len(recs) >= 20
    for r in recs:
        assert B.validate(r)["status"] == "ok", r
    dec = [r for r in recs if r["metric"] == "decode_tok_s" and r["shape"]["tp"] == 1]
    assert dec and dec[0]["floor"] > dec[0]["value"] > 92.4      # above the reference's published figure


def test_memory_plan_optional_rows_and_optimizer_variants():
    cfg = qwen38_27b()
    base = memory.plan(cfg)
    p = memory.plan(cfg, drafter={"width": 8}, indexer={}, host_pages=1000)
    assert {"drafter parameters", "drafter context (per-request K / V)", "page indexer"} <= set(p.rows)
    assert p.blocks < base.blocks                            # the extras come out of what the KV pool gets
    assert any(n.startswith("host KV tier") for n in p.notes)
    assert memory.fit_num_blocks(1000, 100, 0.5) == 5 and memory.fit_num_blocks(-5, 100) == 0
    # the drafter row follows the drafter's real parameter count
    from tilerl_b200.config import tiny_hybrid
    from tilerl_b200.models.hybrid import HybridModel
    from tilerl_b200.spec import BlockDrafter, BlockDrafterConfig
    small = tiny_hybrid()
    dc = BlockDrafterConfig(width=4, n_layers=2, n_heads=4, n_kv_heads=2)
    d = BlockDrafter(HybridModel.build_random(small, seed=0), dc)
    want = sum(t.numel() * t.element_size() for t in d.p.values())
    got = memory.drafter_bytes(small, width=4, n_layers=2, n_heads=4, n_kv_heads=2, taps=len(d.aux_layers))["drafter parameters"]
    assert got == want
    full = {o: memory.train_plan(cfg, mode="full", zero=8, optimizer=o) for o in ("adamw", "adafactor", "iso")}
    assert sum(full["adafactor"].values()) < sum(full["iso"].values()) < sum(full["adamw"].values())
    assert "iso momentum (fp32)" in full["iso"] and "adam moments (fp32 x2)" in full["adamw"]
    with pytest.raises(ValueError):
        memory.train_plan(cfg, optimizer="sgd")


def test_memory_measure_reports_what_a_live_engine_holds():
    import torch
    from helpers import make_engine, rand_prompts
    from tilerl_b200.config import tiny_hybrid
    from tilerl_b200.engine import SamplingParams
    from tilerl_b200.spec import BlockDrafter
    cfg = tiny_hybrid()
    eng = make_engine(cfg, blocks=64)
    eng.drafter = BlockDrafter(eng.model)
    eng.generate(rand_prompts(cfg, 1, 12, seed=1), SamplingParams(max_tokens=3))
    m = memory.measure(eng)
    assert m["kv pool"] == eng.kv.k.numel() * eng.kv.k.element_size() * 2
    assert m["gdn state slots"] >= eng.states.states.numel() * eng.states.states.element_size()
    assert m["weights"] >= sum(t.numel() * t.element_size() for t in eng.model.params.values() if isinstance(t, torch.Tensor))
    assert m["drafter parameters"] == sum(t.numel() * t.element_size() for t in eng.drafter.p.values())
    p = memory.plan(cfg, blocks=64, slots=4)
    table = memory.memory_table(p, measured=m, peak=sum(m.values()))
    assert "measured GiB" in table and "transient" in table


def test_bench_schema_document_lists_the_registry():
    import os
    import re
    doc = open(os.path.join(os.path.dirname(os.path.dirname(__file__)), "docs", "bench-schema.md")).read()
    listed = set(re.findall(r"^\| `([a-z0-9_]+)` \| [^|]+ \| (?:higher|lower) \|", doc, re.M))
    assert listed == set(benchrec.METRICS), listed ^ set(benchrec.METRICS)
    for name, (unit, hib, keys) in benchrec.METRICS.items():
        row = next(ln for ln in doc.splitlines() if ln.startswith(f"| `{name}` |"))
        assert f"| {unit} |" in row and ("higher" if hib else "lower") in row and all(f"`{k}`" in row for k in keys)
    assert str(benchrec.GATE_RATIO) in doc
