"""CLI smoke on CPU: every verb parses and runs its smallest case."""
import json
import os

import pytest

from tilerl_b200 import cli


def test_serve_dry_run_prints_ledger(capsys):
    assert cli.main(["serve", "--model", "qwen38-27b", "--dry-run", "--slots", "16"]) == 0
    out = capsys.readouterr().out
    assert "weights" in out and "kv pool" in out


def test_serve_dry_run_fp8_kv_holds_about_twice_the_tokens(capsys):
    import re
    toks = []
    for fmt in ("bf16", "fp8"):
        assert cli.main(["serve", "--model", "qwen38-27b", "--dry-run", "--slots", "16", "--kv-format", fmt]) == 0
        m = re.search(r"kv pool holds ([\d,]+) tokens", capsys.readouterr().out)
        toks.append(int(m.group(1).replace(",", "")))
    assert 1.9 < toks[1] / toks[0] < 2.0     # one byte per value plus the per-row scales


def test_bench_kernels_table(capsys):
    assert cli.main(["bench", "--model", "qwen38-27b", "--kernels"]) == 0
    out = capsys.readouterr().out
    assert "gate_up" in out and "bound" in out.lower()


def test_bench_registry_lists_the_support_matrix(capsys):
    assert cli.main(["bench", "--registry"]) == 0
    out = capsys.readouterr().out
    assert "gemm_nvfp4_kernel" in out and "sm100" in out and "ref.py" in out


def test_bench_runs_tiny(capsys):
    assert cli.main(["bench", "--model", "tiny", "--device", "cpu", "--prompt-len", "16", "--gen", "4"]) == 0
    rec = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert rec[0]["batch"] == 1 and rec[0]["decode_tok_s"] > 0


def test_train_recipe_and_ledger(tmp_path, capsys):
    runs = str(tmp_path / "runs")
    assert cli.main(["train", "--recipe", "grpo-tiny-smoke", "--device", "cpu", "--steps", "1", "--max-tokens", "4",
                     "--runs", runs, "--prompt-len", "6"]) == 0
    lines = [l for l in capsys.readouterr().out.splitlines() if l.startswith("{")]
    assert json.loads(lines[-1])["step"] == 0
    assert cli.main(["ledger", "--runs", runs]) == 0
    assert "done" in capsys.readouterr().out


def test_train_sft_lora_saves_adapter(tmp_path, capsys):
    out = str(tmp_path / "adapter")
    assert cli.main(["train", "--model", "tiny", "--device", "cpu", "--steps", "1", "--lora-rank", "2",
                     "--save-model", out, "--runs", str(tmp_path / "r"), "--prompt-len", "8"]) == 0
    assert os.path.exists(out)


def test_generate_and_merge(tmp_path, capsys):
    p = tmp_path / "p.jsonl"
    p.write_text('{"prompt": "hi"}\n{"prompt": "yo"}\n')
    assert cli.main(["generate", "--model", "tiny", "--device", "cpu", "--prompts", str(p), "--out",
                     str(tmp_path / "gen"), "--max-tokens", "3"]) == 0
    files = json.loads(capsys.readouterr().out.strip().splitlines()[-1])["files"]
    assert len(open(files[0]).read().splitlines()) == 2


def test_generate_sampling_flags_reach_the_requests(tmp_path, capsys, monkeypatch):
    from tilerl_b200 import engine as eng
    seen = []
    real = eng.SamplingParams

    def spy(**kw):
        seen.append(kw)
        return real(**kw)

    monkeypatch.setattr(eng, "SamplingParams", spy)
    p = tmp_path / "p.jsonl"
    p.write_text('{"prompt": "hi"}\n{"prompt": "yo"}\n{"prompt": "ok"}\n')
    assert cli.main(["generate", "--model", "tiny", "--device", "cpu", "--prompts", str(p), "--out",
                     str(tmp_path / "gen"), "--max-new-tokens", "2", "--temperature", "0.8", "--top-p", "0.9",
                     "--top-k", "5", "--batch", "2"]) == 0
    capsys.readouterr()
    assert len(seen) == 3 and all(k["top_p"] == 0.9 and k["top_k"] == 5 and k["max_tokens"] == 2 for k in seen)
    assert len({k["seed"] for k in seen}) == 3


def test_unknown_recipe():
    with pytest.raises(KeyError):
        cli.main(["train", "--recipe", "nope", "--device", "cpu"])


def test_train_indexer_warmup(tmp_path, capsys):
    out = str(tmp_path / "ix")
    assert cli.main(["train", "--model", "tiny-hybrid", "--indexer-warmup", "--steps", "3", "--ctx", "96",
                     "--save-model", out, "--runs", str(tmp_path / "r"), "--device", "cpu"]) == 0
    rec = json.loads([l for l in capsys.readouterr().out.splitlines() if l.startswith("{")][-1])
    assert rec["steps"] == 3 and os.path.exists(os.path.join(out, "indexer.safetensors"))


def test_train_adapters_with_evals_and_best_adapter(tmp_path, capsys):
    out = str(tmp_path / "ad")
    assert cli.main(["train", "--model", "tiny-hybrid", "--device", "cpu", "--rl", "--lora-rank", "2", "--steps", "3",
                     "--group", "2", "--prompts-per-step", "1", "--max-tokens", "4", "--eval-every", "1",
                     "--patience", "5", "--save-model", out, "--runs", str(tmp_path / "r"), "--prompt-len", "6"]) == 0
    rec = json.loads([l for l in capsys.readouterr().out.splitlines() if l.startswith("{")][-1])
    assert rec["steps"] == 3 and len(rec["evals"]) == 3 and rec["best_eval"] is not None
    assert os.path.exists(os.path.join(out, "adapter.safetensors"))
    assert os.path.exists(os.path.join(out, "adapter-best.safetensors"))


def test_train_deterministic_flag_repeats_the_run(capsys, tmp_path, monkeypatch):
    """Two runs of the tiny GRPO recipe with --deterministic log the same losses."""
    monkeypatch.setenv("TRL_RUNS", str(tmp_path))
    outs = []
    for _ in range(2):
        assert cli.main(["train", "--recipe", "grpo-tiny-smoke", "--device", "cpu", "--deterministic", "--steps", "2",
                         "--force"]) == 0
        lines = [json.loads(ln) for ln in capsys.readouterr().out.splitlines() if ln.startswith("{")]
        outs.append([(ln.get("loss"), ln.get("reward_mean")) for ln in lines if "loss" in ln])
    assert outs[0] and outs[0] == outs[1]


def test_serve_learned_scorer_needs_an_indexer_checkpoint():
    import pytest
    with pytest.raises(SystemExit) as e:
        cli.main(["serve", "--model", "tiny", "--device", "cpu", "--sparse-k", "4", "--scorer", "learned"])
    assert "--indexer" in str(e.value)


def test_bench_suites_are_product_entry_points(capsys):
    """``bench --suite list`` names the measurement suites; each one is an importable module with a
    ``main(argv)`` whose ``--help`` parses (the suites themselves need a GPU)."""
    import importlib
    import pytest
    from tilerl_b200 import suites
    assert cli.main(["bench", "--suite", "list"]) == 0
    names = capsys.readouterr().out.split()
    assert set(names) == set(suites.SUITES) and {"spec", "batch", "sparse", "tick", "grpo", "grpo-zero3"} <= set(names)
    for mod, _ in suites.SUITES.values():
        m = importlib.import_module(f"tilerl_b200.suites.{mod}")
        with pytest.raises(SystemExit) as e:
            m.main(["--help"])
        assert e.value.code == 0
    capsys.readouterr()
    with pytest.raises(SystemExit):
        cli.main(["bench", "--suite", "nope"])
    with pytest.raises(SystemExit):
        cli.main(["bench", "--no-such-flag"])          # unknown flags stay errors outside --suite


def test_bench_record_line_appends_validated_records(tmp_path, monkeypatch, capsys):
    from tilerl_b200 import benchrec
    store = tmp_path / "m.jsonl"
    monkeypatch.setenv("TRL_BENCH_STORE", str(store))
    line = {"metric": "decode_tok_s_b1_27b_nvfp4_prompt512_gen64", "value": 200.0, "n_gpus": 2, "warmup": 3,
            "config": {"model": "qwen38-27b", "prompt_len": 512, "gen_len": 64}, "prefill_tok_s": 9000.0,
            "decode_ms_per_tick": 5.0, "served_bytes": 10_000_000_000,
            "e2e": {"request_tok_s": 150.0, "ttft_ms": 40.0}}
    f = tmp_path / "line.json"
    f.write_text("noise\n" + json.dumps(line) + "\n")
    assert cli.main(["bench", "--record-line", str(f)]) == 0
    recs = benchrec.load(str(store))
    assert {r["metric"] for r in recs} == {"decode_tok_s", "decode_ms_per_tick", "prefill_tok_s", "e2e_request_tok_s", "ttft_ms"}
    assert all(r["status"] == "ok" and r["shape"]["tp"] == 2 for r in recs)


def test_train_rl_on_a_jsonl_of_prompts_and_answers_with_evals_before_and_after(tmp_path, capsys, monkeypatch):
    """GRPO on real prompts: --data gives {prompt, answer} rows (the reward is an exact match of the last
    number of the completion), --eval-gsm8k scores greedy accuracy before and after, --lineage records the
    parent run, --length-penalty reaches the loop."""
    monkeypatch.setenv("TRL_RUNS", str(tmp_path / "runs"))
    data = tmp_path / "train.jsonl"
    data.write_text("\n".join(json.dumps({"prompt": f"{a}+{b}=", "answer": str(a + b)}) for a, b in ((1, 2), (3, 4), (2, 2), (5, 1))))
    ev = tmp_path / "eval.jsonl"
    ev.write_text("\n".join(json.dumps({"question": f"{a}+{a}=", "answer": str(2 * a)}) for a in (1, 2, 3)))
    assert cli.main(["train", "--model", "tiny", "--device", "cpu", "--rl", "--steps", "1", "--group", "2",
                 "--prompts-per-step", "2", "--max-tokens", "4", "--data", str(data), "--eval-gsm8k", str(ev),
                 "--eval-n", "2", "--eval-max-new-tokens", "4", "--length-penalty", "0.01", "--lineage", "abc123"]) == 0
    out = [json.loads(ln) for ln in capsys.readouterr().out.splitlines() if ln.startswith("{")]
    assert "eval_before" in out[0] and out[0]["eval_before"]["n"] == 2
    assert "eval_after" in out[-1] and 0.0 <= out[-1]["eval_after"]["accuracy"] <= 1.0
    steps = [o for o in out if "reward" in o or "mean_reward" in o]
    assert len(steps) == 1
    runs = os.listdir(tmp_path / "runs")
    man = json.load(open(tmp_path / "runs" / runs[0] / "manifest.json"))
    assert man["parent"] == "abc123" and man["inputs"]["data"] == str(data)
    assert any("eval_before_accuracy" in m for m in man["metrics"])


def test_train_dry_run_prints_the_training_memory_plan_and_ledger_reads_time_to_score(tmp_path, capsys):
    assert cli.main(["train", "--model", "qwen38-27b", "--dry-run", "--optim", "adafactor", "--zero", "8",
                     "--train-seq-len", "4096"]) == 0
    out = capsys.readouterr().out
    assert "fp32 master" in out and "adafactor second moment" in out and "total" in out
    assert cli.main(["train", "--model", "qwen38-27b", "--dry-run", "--lora-rank", "16"]) == 0
    assert "adapters (fp32)" in capsys.readouterr().out
    from tilerl_b200 import ledger
    r = ledger.Run({"cmd": "train"}, root=str(tmp_path))
    r.log(step=0, eval_reward=0.1)
    r.log(step=1, eval_reward=0.6)
    r.finish()
    assert cli.main(["ledger", "--runs", str(tmp_path), "--time-to-score", "0.5"]) == 0
    line = capsys.readouterr().out.strip().splitlines()[-1]
    assert "eval_reward>=0.5:" in line and "never" not in line
    assert cli.main(["ledger", "--runs", str(tmp_path), "--time-to-score", "0.9"]) == 0
    assert "never" in capsys.readouterr().out


def test_spill_file_capacity_follows_the_flag_or_the_free_space(tmp_path):
    assert cli.ssd_slots(str(tmp_path / "spill.bin"), 10 * 4096, 4096) == 10
    assert cli.ssd_slots(str(tmp_path / "spill.bin"), 100, 4096) == 1
    free = cli.ssd_slots(str(tmp_path / "spill.bin"), 0, 1 << 20)
    assert 1 <= free <= 1 << 24
    args = cli.build_parser().parse_args(["serve", "--cold-ssd-path", "x", "--cold-ssd-bytes", "123", "--stream-pace-depth", "12"])
    assert args.cold_ssd_bytes == 123 and args.stream_pace_depth == 12


def test_text_reward_recipes_need_gold_answers():
    with pytest.raises(SystemExit) as e:
        cli.main(["train", "--recipe", "grpo-gsm8k-27b", "--device", "cpu", "--steps", "1"])
    assert "--data" in str(e.value)


def test_train_hands_back_a_finished_run_and_force_trains_again(capsys, tmp_path, monkeypatch):
    monkeypatch.setenv("TRL_RUNS", str(tmp_path))
    cmd = ["train", "--recipe", "grpo-tiny-smoke", "--device", "cpu", "--steps", "1", "--seed", "11"]
    assert cli.main(cmd) == 0
    first = [json.loads(ln) for ln in capsys.readouterr().out.splitlines() if ln.startswith("{")]
    assert any("loss" in ln for ln in first)
    assert cli.main(cmd) == 0                                   # the same inputs: the same run, already done
    again = [json.loads(ln) for ln in capsys.readouterr().out.splitlines() if ln.startswith("{")]
    assert len(again) == 1 and again[0]["reused"] is True and again[0]["status"] == "done"
    assert cli.main(cmd + ["--json"]) == 0                      # --json: the whole manifest
    man = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert man["id"] == again[0]["run"] and man["inputs"]["seed"] == 11 and man["metrics"]
    assert cli.main(cmd + ["--force", "--json"]) == 0           # trained again: one line, the fresh manifest
    out = [ln for ln in capsys.readouterr().out.splitlines() if ln.startswith("{")]
    assert len(out) == 1 and json.loads(out[0])["id"] == man["id"] and json.loads(out[0])["status"] == "done"
    assert cli.main(cmd[:-1] + ["12"]) == 0                     # another seed is another run
    other = [json.loads(ln) for ln in capsys.readouterr().out.splitlines() if ln.startswith("{")]
    assert any("loss" in ln for ln in other)


def test_rollout_length_guards():
    from tilerl_b200 import rl
    rl.refuse_short_rollouts(None, 512)                       # nothing measured: nothing to compare
    rl.refuse_short_rollouts(300.0, 512)                      # 300 <= 0.8 * 512
    rl.refuse_short_rollouts(1038.0, 512, allow=True)
    with pytest.raises(SystemExit) as e:
        rl.refuse_short_rollouts(1038.0, 512)
    assert "1038" in str(e.value) and "1298" in str(e.value) and "--allow-short-rollouts" in str(e.value)
    d = rl.RolloutDrift(cap=100)
    assert all(d.update(95.0, i + 1) for i in range(4))       # fewer than five steps: no verdict yet
    assert d.update(20.0, 5) is True and d.mean == pytest.approx(80.0)        # (4 * 95 + 20) / 5 = 80 <= 80
    assert d.update(95.0, 6) is True and d.mean == pytest.approx(80.0)        # the window is the last five
    d2 = rl.RolloutDrift(cap=100)
    for i in range(5):
        ok = d2.update(90.0, i + 1)
    assert ok is False and "average 90.0" in d2.reason and "above 112" in d2.reason


def test_train_stops_when_rollouts_run_into_the_cap(capsys, tmp_path, monkeypatch):
    # the tiny random policy never ends by itself: every rollout runs to the cap, and the sixth step never starts
    monkeypatch.setenv("TRL_RUNS", str(tmp_path))
    cmd = ["train", "--rl", "--model", "tiny", "--device", "cpu", "--steps", "8", "--max-tokens", "4", "--group", "2",
           "--prompts-per-step", "1", "--seed", "5"]
    assert cli.main(cmd) == 1
    cap = capsys.readouterr()
    steps = [json.loads(ln) for ln in cap.out.splitlines() if ln.startswith("{") and "loss" in ln]
    assert len(steps) == 5 and "rollout cap is 4" in cap.err
    assert cli.main(cmd + ["--allow-short-rollouts"]) == 0
    steps = [json.loads(ln) for ln in capsys.readouterr().out.splitlines() if ln.startswith("{") and "loss" in ln]
    assert len(steps) == 8


def test_train_curve_subset_mmlu_arm_and_rollout_rows(tmp_path, capsys, monkeypatch):
    monkeypatch.setenv("TRL_RUNS", str(tmp_path / "runs"))
    data = tmp_path / "train.jsonl"
    data.write_text("\n".join(json.dumps({"prompt": f"{a}+{b}=", "answer": str(a + b)}) for a, b in ((1, 2), (3, 4))))
    ev = tmp_path / "eval.jsonl"
    ev.write_text("\n".join(json.dumps({"question": f"{a}+{a}=", "answer": str(2 * a)}) for a in range(1, 9)))
    mm = tmp_path / "mmlu.jsonl"
    mm.write_text("\n".join(json.dumps({"question": f"q{i}?", "choices": ["w", "x", "y", "z"], "answer": "B"}) for i in range(3)))
    base = ["train", "--model", "tiny", "--device", "cpu", "--rl", "--steps", "2", "--group", "2", "--prompts-per-step", "1",
            "--max-tokens", "4", "--data", str(data), "--eval-gsm8k", str(ev), "--eval-n", "2", "--eval-max-new-tokens", "4",
            "--eval-every", "1", "--allow-short-rollouts"]
    with pytest.raises(SystemExit) as e:                        # 4 rows: SE 25 pt against a 5 pt effect
        cli.main(base + ["--eval-curve-n", "4"])
    assert "25.0 pt" in str(e.value) and ">=100" in str(e.value)
    assert cli.main(base + ["--eval-curve-n", "4", "--curve-target-pt", "30", "--eval-mmlu", str(mm)]) == 0
    out = [json.loads(ln) for ln in capsys.readouterr().out.splitlines() if ln.startswith("{")]
    curve = [o for o in out if "curve_step" in o]
    assert [c["curve_step"] for c in curve] == [0, 1, 2] and all(c["curve_n"] == 4 and "curve_se_pt" in c for c in curve)
    assert sum("mmlu_before" in o for o in out) == 1 and sum("mmlu_after" in o for o in out) == 1
    assert next(o for o in out if "mmlu_before" in o)["mmlu_before"]["n"] == 2       # --eval-n rows
    run = os.listdir(tmp_path / "runs")[0]
    rows = [json.loads(ln) for ln in open(tmp_path / "runs" / run / "rollouts.jsonl")]
    assert len(rows) == 4 and {r["step"] for r in rows} == {0, 1}          # steps x group x prompts
    assert all({"tokens", "reward", "task", "finish", "prompt"} <= set(r) for r in rows)
    man = json.load(open(tmp_path / "runs" / run / "manifest.json"))
    assert not any("rollouts" in m for m in man["metrics"]) and any("curve_accuracy" in m for m in man["metrics"])
    from tilerl_b200 import ledger
    a, b = ledger.curve_rows(list(range(50)), 10, 0), ledger.curve_rows(list(range(50)), 10, 0)
    assert a == b and a != list(range(10)) and len(set(a)) == 10       # a fixed shuffle, not the head of the file
    assert ledger.binomial_se_pt(0.5, 100) == pytest.approx(5.0) and ledger.binomial_se_pt(1.0, 10) == 0.0
    ledger.refuse_blind_curve(100, 5.0)                                   # SE exactly at the target passes


def test_serve_dry_run_json_against_a_given_free_size_and_state_budget(capsys):
    assert cli.main(["serve", "--model", "qwen38-27b", "--dry-run", "--slots", "16", "--json"]) == 0
    whole = json.loads(capsys.readouterr().out)
    assert whole["rows"]["weights"] > 10 << 30 and whole["total_static"] == sum(whole["rows"].values())
    assert whole["free_after"] == whole["device_bytes"] - whole["total_static"] and whole["blocks"] > 0
    assert cli.main(["serve", "--model", "qwen38-27b", "--dry-run", "--slots", "16", "--json", "--device-free",
                     str(80 << 30), "--state-bytes", str(3 << 30)]) == 0
    part = json.loads(capsys.readouterr().out)
    assert part["device_bytes"] == 80 << 30 and part["rows"]["prefix state store"] == 3 << 30
    assert 0 < part["blocks"] < whole["blocks"] and part["rows"]["weights"] == whole["rows"]["weights"]


def test_bench_kernels_takes_a_context_a_prefill_length_and_a_device_name(capsys):
    assert cli.main(["bench", "--model", "qwen38-27b", "--kernels", "--context", "32768", "--device-name", "h20"]) == 0
    out = capsys.readouterr().out
    assert out.startswith("# floors (nominal): 4000 GB/s") and "attn.paged" in out
    paged = next(ln for ln in out.splitlines() if ln.startswith("attn.paged"))
    assert float(paged.split()[-5]) > 2000                # 16 layers x 134 MB of K / V at a 32 768-token context
    assert cli.main(["bench", "--model", "qwen38-27b", "--kernels", "--prefill", "2048"]) == 0
    out = capsys.readouterr().out
    assert "lm_head (last token)" in out and "gdn.step" not in out          # the prefill table alone
    with pytest.raises(SystemExit) as e:
        cli.main(["bench", "--model", "qwen38-27b", "--kernels", "--device-name", "tpu"])
    assert "no floor known" in str(e.value)
    from tilerl_b200.calibration import peaks_for
    assert peaks_for("NVIDIA B200").source in ("measured", "fallback") and peaks_for("V100-SXM2").hbm_gbs == 900.0


def test_train_indexer_corpus_run_reports_recall_per_length_and_a_control(tmp_path, capsys, monkeypatch):
    import torch
    monkeypatch.setenv("TRL_RUNS", str(tmp_path / "runs"))
    g = torch.Generator().manual_seed(0)

    def spans(d, split, ctx, n):
        os.makedirs(d, exist_ok=True)
        with open(os.path.join(d, f"{split}_{ctx}.jsonl"), "w") as f:
            for _ in range(n):
                f.write(json.dumps({"ctx": ctx, "ids": torch.randint(0, 200, (ctx,), generator=g).tolist()}) + "\n")
    main_dir, ctl = str(tmp_path / "corpus"), str(tmp_path / "control")
    for ctx in (96, 128, 160):
        spans(main_dir, "train", ctx, 2)
        spans(main_dir, "held", ctx, 3)
    spans(ctl, "held", 96, 1)
    from tilerl_b200.sparse_index import load_spans
    cut = load_spans(main_dir, "held", 4)                      # 4 spans over three lengths: 2 / 1 / 1
    assert {k: len(v) for k, v in cut.items()} == {"128": 1, "160": 1, "96": 1} | {sorted(cut)[0]: 2}
    assert cli.main(["train", "--model", "tiny-hybrid", "--indexer-warmup", "--indexer-corpus", main_dir,
                     "--indexer-control-corpus", ctl, "--steps", "4", "--k-pages", "2", "--q-samples", "4",
                     "--held-spans", "4", "--indexer-di", "32", "--save-model", str(tmp_path / "ix")]) == 0
    out = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert set(out["recall_before"]) == set(out["recall_after"]) == {"96", "128", "160"}
    assert all(0.0 < v <= 1.0 for v in out["recall_after"].values()) and out["di"] == 32 and out["k_pages"] == 2
    assert set(out["control"]["recall_after"]) == {"96"} and out["tokens_seen"] > 0 and out["passed"] is True
    assert os.path.exists(tmp_path / "ix" / "indexer.safetensors")
    # the gate: a threshold no indexer reaches fails the run
    assert cli.main(["train", "--model", "tiny-hybrid", "--indexer-warmup", "--indexer-corpus", main_dir, "--steps", "1",
                     "--k-pages", "1", "--q-samples", "2", "--held-spans", "3", "--recall-threshold", "1.01"]) == 1
    man = [json.load(open(tmp_path / "runs" / d / "manifest.json")) for d in os.listdir(tmp_path / "runs")]
    assert sorted(m["status"] for m in man) == ["done", "gate_failed"]


def test_merge_is_a_run_whose_parents_are_the_runs_that_wrote_its_inputs(tmp_path, capsys, monkeypatch):
    runs = str(tmp_path / "runs")
    monkeypatch.setenv("TRL_RUNS", runs)
    outs = []
    for seed in ("1", "2", "3"):             # a base and two "specialists": full-parameter runs that save a checkpoint
        out = str(tmp_path / f"ckpt{seed}")
        assert cli.main(["train", "--model", "tiny", "--device", "cpu", "--steps", "1", "--seed", seed, "--prompt-len", "8",
                         "--save-model", out]) == 0
        outs.append(out)
    capsys.readouterr()
    merged = str(tmp_path / "merged")
    cmd = ["merge", "--base", outs[0], "--specialists", f"{outs[1]},{outs[2]}", "--out", merged, "--method", "ties"]
    assert cli.main(cmd) == 0
    rec = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert rec["tensors"] > 0 and len(rec["parents"]) == 3 and os.path.isdir(merged)
    from tilerl_b200 import ledger
    man = ledger.load_run(rec["run"], runs)
    assert man["status"] == "done" and man["parents"] == rec["parents"] and man["artifacts"]["model"] == merged
    assert all(ledger.load_run(p, runs)["inputs"]["cmd"] == "train" for p in man["parents"])
    assert ledger.find_run_for_artifact(str(tmp_path / "nowhere"), runs) is None
    assert ledger.find_run_for_artifact(merged, runs) == rec["run"]
    assert cli.main(cmd) == 0                                   # the same merge asked again: the finished run
    assert json.loads(capsys.readouterr().out.strip().splitlines()[-1])["reused"] is True
    assert cli.main(cmd + ["--force", "--json"]) == 0
    assert json.loads(capsys.readouterr().out.strip().splitlines()[-1])["id"] == rec["run"]
    with pytest.raises(SystemExit):
        cli.main(["merge", "--base", outs[0], "--out", merged])


def test_serve_records_residency_and_the_devices_ledger_reads_it(tmp_path, capsys, monkeypatch):
    store = tmp_path / "bench.jsonl"
    monkeypatch.setenv("TRL_BENCH_STORE", str(store))
    assert cli.main(["serve", "--model", "tiny", "--device", "cpu", "--slots", "4", "--blocks", "64", "--no-warmup",
                     "--record-residency", "--port", "0"]) == 0
    res = json.loads(capsys.readouterr().out.strip().splitlines()[-1])["residency"]
    assert res["static"] > 0 and res["peak"] >= res["static"] and res["transient"] == res["peak"] - res["static"]
    from tilerl_b200 import benchrec, ledger
    recs = benchrec.load(str(store))
    assert {r["metric"] for r in recs} >= {"resident_peak_bytes", "resident_static_bytes"}
    assert all(r["shape"] == {"model": "tiny", "slots": 4, "tp": 1} and r["unit"] == "B" for r in recs)
    benchrec.append(benchrec.make_record("hbm_copy_gbs", 6850.0, {}, target="b200"), str(store))
    benchrec.append(benchrec.make_record("bf16_gemm_tflops", 1590.0, {}, target="b200"), str(store))
    secs = {s["device"]: s for s in ledger.device_sections(benchrec.load(str(store)))}
    assert secs["cpu"]["residency"]["peak"] == res["peak"] and secs["cpu"]["hbm_copy_gbs"] is None
    assert secs["b200"]["hbm_copy_gbs"]["value"] == 6850.0 and secs["b200"]["residency"] is None
    assert cli.main(["ledger", "--devices"]) == 0
    out = capsys.readouterr().out
    assert "hbm_copy_gbs 6850.0" in out and "resident" in out and "none recorded (run serve --record-residency)" in out


def test_serve_draft_window_flag_reaches_the_plan(capsys, monkeypatch):
    def ctx_gib(extra):
        assert cli.main(["serve", "--model", "qwen38-27b", "--dry-run", "--slots", "16", "--draft", "block", "--json"] + extra) == 0
        rows = json.loads(capsys.readouterr().out)["rows"]
        return next(v for k, v in rows.items() if "drafter context" in k)
    base = ctx_gib([])
    assert ctx_gib(["--draft-attn-window-tokens", "128"]) == 2 * base          # default window 64
    monkeypatch.setenv("TRL_DRAFT_ATTN_WINDOW_TOKENS", "32")
    assert ctx_gib([]) * 2 == base and ctx_gib(["--draft-attn-window-tokens", "64"]) == base      # the flag wins


def test_a_run_that_loads_an_adapter_descends_from_the_run_that_wrote_it(tmp_path, capsys, monkeypatch):
    runs = str(tmp_path / "runs")
    monkeypatch.setenv("TRL_RUNS", runs)
    out = str(tmp_path / "adapter")
    base = ["train", "--model", "tiny", "--device", "cpu", "--steps", "1", "--lora-rank", "2", "--prompt-len", "8"]
    assert cli.main(base + ["--save-model", out]) == 0
    from tilerl_b200 import ledger
    first = ledger.list_runs(runs)
    assert len(first) == 1 and first[0]["artifacts"]["model"] == out
    assert cli.main(base + ["--load-adapter", out, "--seed", "3"]) == 0
    capsys.readouterr()
    child = [r for r in ledger.list_runs(runs) if r["id"] != first[0]["id"]]
    assert len(child) == 1 and child[0]["parent"] == first[0]["id"]
    assert ledger.lineage(child[0]["id"], runs) == [child[0]["id"], first[0]["id"]]
