"""Engine integration on the tiny hybrid config (CPU, fp32): the served tokens
must equal an unfused full-sequence fp32 forward, however the work is chunked,
batched, cached or speculated."""
import torch

from helpers import autograd_forward, make_engine, rand_prompts
from tilerl_b200.config import tiny, tiny_hybrid
from tilerl_b200.engine import EngineOverloaded, SamplingParams, StepLimits
from tilerl_b200.kv import PrefixStore


def dense_greedy(model, prompt, n):
    seq = list(prompt)
    with torch.no_grad():
        for _ in range(n):
            lg = autograd_forward(model, torch.tensor([seq]), {})
            seq.append(int(lg[0, -1].argmax()))
    return seq[len(prompt):]


def test_config1_serve_matches_unfused_fp32():
    cfg = tiny_hybrid()
    eng = make_engine(cfg)
    prompts = rand_prompts(cfg, 2, 32)
    res = eng.generate(prompts, SamplingParams(max_tokens=16))
    for p, r in zip(prompts, res):
        assert r.tokens == dense_greedy(eng.model, p, 16)
        assert r.finish_reason == "length" and r.prompt_tokens == 32


def test_chunked_prefill_equals_one_shot_and_batch_equals_single():
    cfg = tiny_hybrid()
    prompts = rand_prompts(cfg, 3, 45, seed=5)
    one = make_engine(cfg, limits=StepLimits(max_batched_tokens=512))
    ref_out = [one.generate([p], SamplingParams(max_tokens=6))[0].tokens for p in prompts]
    chunked = make_engine(cfg, limits=StepLimits(max_batched_tokens=16, prefill_align=8))
    got = chunked.generate(prompts, SamplingParams(max_tokens=6))
    assert [r.tokens for r in got] == ref_out
    assert chunked.counters["mixed_ticks"] + chunked.counters["prefill_ticks"] > 3


def test_prefix_hit_equals_cold():
    cfg = tiny_hybrid()
    eng = make_engine(cfg)
    eng.prefix = PrefixStore(eng.kv)
    p = rand_prompts(cfg, 1, 40, seed=9)[0]
    cold = eng.generate([p], SamplingParams(max_tokens=5))[0]
    warm = eng.generate([p], SamplingParams(max_tokens=5))[0]
    assert warm.tokens == cold.tokens
    assert eng.prefix.hits == 1 and warm.cached_tokens == 32
    longer = p[:36] + [7, 8, 9]
    fresh = make_engine(cfg).generate([longer], SamplingParams(max_tokens=5))[0]
    assert eng.generate([longer], SamplingParams(max_tokens=5))[0].tokens == fresh.tokens
    eng.invalidate_weights()
    assert len(eng.prefix) == 0 and eng.kv.used_blocks == 0


def test_seeded_sampling_is_reproducible_and_logprobs_returned():
    cfg = tiny()
    eng = make_engine(cfg)
    p = rand_prompts(cfg, 1, 12)[0]
    sp = SamplingParams(max_tokens=8, temperature=1.0, top_p=0.9, seed=11, logprobs=True)
    a = eng.generate([p], sp)[0]
    b = eng.generate([p], sp)[0]
    assert a.tokens == b.tokens and len(a.logprobs) == 8 and all(l <= 0 for l in a.logprobs)
    c = eng.generate([p], SamplingParams(max_tokens=8, temperature=1.0, top_p=0.9, seed=12))[0]
    assert c.tokens != a.tokens


def test_stop_ids_cancel_overload_and_pool_release():
    cfg = tiny()
    eng = make_engine(cfg, limits=StepLimits(max_inflight=2))
    p = rand_prompts(cfg, 1, 10)[0]
    first = eng.generate([p], SamplingParams(max_tokens=4))[0].tokens
    r = eng.generate([p], SamplingParams(max_tokens=10, stop_ids=(first[1],)))[0]
    assert r.finish_reason == "stop" and r.tokens == first[:first.index(first[1]) + 1]
    a = eng.submit(p, SamplingParams(max_tokens=50))
    b = eng.submit(p, SamplingParams(max_tokens=50))
    try:
        eng.submit(p)
        assert False, "expected overload"
    except EngineOverloaded:
        pass
    eng.step()
    assert eng.cancel(a) and eng.take(a).finish_reason == "cancelled"
    while eng.poll(b)["state"] != "done":
        eng.step()
    assert eng.kv.used_blocks == 0 and eng.states.free_slots == eng.states.num_slots - 1


def test_daemon_loop_and_peek():
    import time
    cfg = tiny()
    eng = make_engine(cfg)
    eng.run(batching_window_s=0.0)
    rid = eng.submit(rand_prompts(cfg, 1, 8)[0], SamplingParams(max_tokens=5))
    for _ in range(400):
        toks, done = eng.peek(rid)
        if done:
            break
        time.sleep(0.01)
    eng.stop()
    assert done and len(eng.take(rid).tokens) == 5
    assert eng.liveness()["last_progress_age_s"] == 0.0


def test_fp8_kv_pool_serves_close_to_bf16_and_halves_the_pool():
    """fp8 KV (e4m3 + one fp32 scale per token and head): same greedy tokens on the tiny model's
    first steps, logits within the fp8 rounding, pool bytes per block ~half of fp32/2."""
    import torch
    from tilerl_b200.batch import Batch
    from tilerl_b200.kv import GdnStatePool, PagedKvPool
    from tilerl_b200.models.hybrid import HybridModel
    from tilerl_b200.ops.backend import RefOps
    cfg = tiny_hybrid()
    model = HybridModel.build_random(cfg, seed=2)
    ops = RefOps()
    outs = []
    for fp8 in (False, True):
        kv = PagedKvPool(cfg, 8, dtype=torch.float32, fp8=fp8)
        st = GdnStatePool(cfg, 4, ring_dtype=torch.float32)
        seqs = [dict(tokens=list(range(3, 27)), start=0, blocks=[1, 2], slot=1)]
        lg1 = model.forward(Batch.build(seqs, "cpu"), ops, kv, st).float().clone()
        lg2 = model.forward(Batch.build([dict(tokens=[5], start=24, blocks=[1, 2], slot=1)], "cpu"), ops, kv, st).float()
        outs.append((lg1, lg2.clone(), kv.block_bytes()))
    rel = float((outs[1][1] - outs[0][1]).norm() / outs[0][1].norm())
    assert 0 < rel < 0.05, rel
    assert outs[1][0].argmax(-1).tolist() == outs[0][0].argmax(-1).tolist()
    assert outs[1][2] < 0.4 * outs[0][2]            # fp8 + scales vs the fp32 oracle pool
    k, v = kv.read_block(1)
    kv.write_block(3, k, v)
    k2, _ = kv.read_block(3)
    assert float((k2 - k).abs().max()) <= 0.07 * float(k.abs().max()) + 1e-6


def test_poisoned_pools_give_the_same_tokens():
    """Reads of unwritten pool memory would show: with every KV page, GDN state and conv ring
    filled with NaN before the first request, the tokens equal those of zero-filled pools."""
    from tilerl_b200.engine import SamplingParams
    cfg = tiny_hybrid()
    prompts = rand_prompts(cfg, 3, 21)
    outs = []
    for poison in (False, True):
        eng = make_engine(cfg, planes=1)
        if poison:
            for t in (eng.kv.k, eng.kv.v, eng.states.states, eng.states.ring):
                t.fill_(float("nan"))
        outs.append([r.tokens for r in eng.generate(prompts, SamplingParams(max_tokens=10))])
    assert outs[0] == outs[1]


def test_batched_sampler_seam_gets_every_sampling_row_of_a_tick():
    """A backend that offers ``sample_rows`` receives, in one call per tick, every row that samples
    (plain temperature, top-k, top-p) with its seed stream and restrictions; greedy rows and rows
    with an allowed-id list stay on their own paths; tokens equal the per-row host sampler's."""
    from tilerl_b200.engine import SamplingParams
    from tilerl_b200.ops import ref
    from tilerl_b200.ops.backend import RefOps

    calls = []

    class Ops(RefOps):
        def sample_rows(self, logits, rows, seeds, temps, top_ks=None, top_ps=None):
            calls.append((list(rows), list(top_ks), list(top_ps)))
            out = [ref.sample(logits[r].detach().float().cpu(), t, p, k, s)
                   for r, s, t, k, p in zip(rows, seeds, temps, top_ks, top_ps)]
            return [o[0] for o in out], [o[1] for o in out]

    cfg = tiny_hybrid()
    prompts = rand_prompts(cfg, 4, 9)
    params = [SamplingParams(max_tokens=6, temperature=1.0, seed=1),
              SamplingParams(max_tokens=6, temperature=0.8, top_k=5, top_p=0.9, seed=2),
              SamplingParams(max_tokens=6),
              SamplingParams(max_tokens=6, temperature=1.0, allowed_ids=(1, 2, 3, 4), seed=3)]
    want = [r.tokens for r in make_engine(cfg).generate(prompts, params)]
    eng = make_engine(cfg)
    eng.ops = Ops()
    got = [r.tokens for r in eng.generate(prompts, params)]
    assert got == want
    assert calls and all(len(c[0]) == 2 for c in calls)          # the two sampling rows, never the other two
    assert all(c[1] == [0, 5] and c[2] == [1.0, 0.9] for c in calls)
    assert all(t in (1, 2, 3, 4) for t in got[3])


def test_pool_exhaustion_preempts_the_newest_request_and_recomputes_it_without_changing_its_output():
    """Two requests that cannot both grow to their full length in a small KV pool: the newer one gives its
    pages back, waits, is recomputed by a prefill over prompt + generated tokens and finishes with exactly
    the tokens it produces when memory is plentiful (greedy and seeded sampling); nothing leaks."""
    cfg = tiny_hybrid()
    prompts = rand_prompts(cfg, 2, 20, seed=11)
    for sp in (SamplingParams(max_tokens=44), SamplingParams(max_tokens=44, temperature=1.0, top_p=0.9, seed=3)):
        roomy = make_engine(cfg, blocks=64)
        want = [r.tokens for r in roomy.generate(prompts, sp)]
        assert roomy.counters["preempted"] == 0
        tight = make_engine(cfg, model=roomy.model, blocks=7)      # 6 usable pages: one request alone needs 4, then 5
        got = tight.generate(prompts, sp)
        assert [r.tokens for r in got] == want
        assert all(r.finish_reason == "length" and len(r.tokens) == 44 for r in got)
        assert tight.counters["preempted"] >= 1 and tight.counters["failed"] == 0
        assert tight.kv.used_blocks == 0 and tight.states.free_slots == roomy.states.free_slots
    # a request that cannot fit even alone is still cut short rather than spinning
    lone = make_engine(cfg, model=roomy.model, blocks=3)
    res = lone.generate(prompts[:1], SamplingParams(max_tokens=44))[0]
    assert res.finish_reason in ("length", "error") and len(res.tokens) < 44


def test_long_fill_cap_bounds_the_prefill_chunk_only_while_the_engine_is_shared():
    cfg = tiny_hybrid()
    long_p, short_p = rand_prompts(cfg, 1, 200, seed=21)[0], rand_prompts(cfg, 1, 20, seed=22)[0]
    limits = StepLimits(max_batched_tokens=128, prefill_align=8, long_prefill_cap=16, long_prefill_min=100)
    eng = make_engine(cfg, limits=limits, blocks=128)
    ref_long = make_engine(cfg, blocks=128).generate([long_p], SamplingParams(max_tokens=4))[0].tokens
    ref_short = make_engine(cfg, blocks=128).generate([short_p], SamplingParams(max_tokens=4))[0].tokens
    # alone in the engine the fill takes the whole budget: 200 tokens in two ticks
    alone = make_engine(cfg, limits=limits, blocks=128)
    rid = alone.submit(long_p, SamplingParams(max_tokens=4))
    alone.step()
    assert alone._reqs[rid].n_computed == 128
    # shared: the long fill advances 16 tokens per tick, the short request prefills beside it and finishes first
    a = eng.submit(long_p, SamplingParams(max_tokens=4))
    b = eng.submit(short_p, SamplingParams(max_tokens=4))
    eng.step()
    assert eng._reqs[a].n_computed == 16 and eng._reqs[b].n_computed == 20
    ticks = 1
    while eng._reqs[b].state != "done":
        eng.step()
        ticks += 1
    assert ticks <= 6 and eng._reqs[a].state == "prefill" and eng._reqs[a].n_computed <= 16 * ticks
    eng.step()                             # alone again: the cap lifts
    assert eng._reqs[a].n_computed >= 16 * ticks + 100 or eng._reqs[a].state != "prefill"
    while eng._reqs[a].state != "done":
        eng.step()
    assert eng.take(a).tokens == ref_long and eng.take(b).tokens == ref_short


def test_stats_report_tick_kinds_memory_rows_and_prefix_traffic():
    cfg = tiny_hybrid()
    eng = make_engine(cfg)
    eng.prefix = PrefixStore(eng.kv)
    p = rand_prompts(cfg, 1, 40, seed=2)[0]
    eng.generate([p], SamplingParams(max_tokens=4))
    s = eng.stats()
    assert s["dense_ticks"] == s["ticks"] > 0 and s["sparse_ticks"] == 0 and s["verify_ticks"] == 0
    assert s["memory"]["kv pool"] > 0 and s["memory"]["weights"] > 0 and s["memory"]["gdn state slots"] > 0
    assert s["prefix_state_bytes"] > 0 and s["spec_acceptance"] is None and s["prefix_promotions"] == 0
    import json
    json.dumps(s)                      # the health route serialises it
