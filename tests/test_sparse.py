"""Sparse KV: top-k >= pages equals dense; selection finds the page that matters; refresh
cadence; dense below the threshold."""
import torch

from helpers import make_engine, rand_prompts
from tilerl_b200.config import tiny_hybrid
from tilerl_b200.engine import SamplingParams
from tilerl_b200.sparse import SparseConfig, SparseKV, learned_index_scores, quest_scores, select_pages


def test_select_pages_device_form():
    s = torch.tensor([0.1, 5.0, 0.2, 4.0, 0.0, 0.0, 0.0, 0.0])
    assert select_pages(s, 8, top_k=2, window=3).tolist() == [1, 3, 5, 6, 7]
    assert select_pages(s, 2, top_k=4, window=3).tolist() == [0, 1]


def test_quest_bound_dominates_true_scores_and_finds_planted_page():
    torch.manual_seed(0)
    hq, hkv, d, pages = 4, 2, 16, 10
    k = torch.randn(pages, hkv, 16, d) * 0.1
    q = torch.randn(hq, d)
    k[6, :, 3] = q.view(hkv, 2, d).mean(1) * 3        # page 6 holds keys aligned with the query
    bounds = torch.stack([k.amin(2), k.amax(2)], dim=2)
    sc = quest_scores(q, bounds)
    true = torch.einsum("hgd,phtd->phgt", q.view(hkv, 2, d), k).amax(-1).sum((1, 2))
    assert (sc >= true - 1e-5).all() and int(sc.argmax()) == 6
    li = learned_index_scores(torch.randn(4, 8), torch.randn(pages, 4, 8))
    assert li.shape == (pages,) and (li >= 0).all()


def test_sparse_with_k_covering_everything_equals_dense_and_refresh_counts():
    cfg = tiny_hybrid()
    prompts = rand_prompts(cfg, 2, 70, seed=6)
    sp = SamplingParams(max_tokens=12)
    dense = make_engine(cfg, blocks=200)
    want = [r.tokens for r in dense.generate(prompts, sp)]
    mgr = SparseKV(cfg, SparseConfig(top_k=64, window=2, refresh_ticks=4, min_tokens=32))
    eng = make_engine(cfg, blocks=200, model=dense.model, sparse=mgr)
    assert [r.tokens for r in eng.generate(prompts, sp)] == want
    assert mgr.stats["sparse_ticks"] >= 10 and 2 <= mgr.stats["refreshes"] <= 8
    # below the threshold: dense ticks only
    mgr2 = SparseKV(cfg, SparseConfig(min_tokens=10_000))
    eng2 = make_engine(cfg, blocks=200, model=dense.model, sparse=mgr2)
    assert [r.tokens for r in eng2.generate(prompts, sp)] == want and mgr2.stats["sparse_ticks"] == 0


def test_truly_sparse_run_is_well_formed():
    cfg = tiny_hybrid()
    mgr = SparseKV(cfg, SparseConfig(top_k=1, window=1, refresh_ticks=2, min_tokens=16))
    eng = make_engine(cfg, blocks=200, sparse=mgr)
    out = eng.generate(rand_prompts(cfg, 1, 90, seed=2), SamplingParams(max_tokens=6))[0]
    assert len(out.tokens) == 6 and eng.kv.used_blocks == 0 and not mgr._sel


def test_learned_indexer_warmup_lowers_the_kl_to_the_dense_page_mass():
    import torch
    from tilerl_b200.config import tiny_hybrid
    from tilerl_b200.models.hybrid import HybridModel
    from tilerl_b200.sparse_index import LearnedIndexer, page_mass, topk_recall, warmup
    cfg = tiny_hybrid()
    model = HybridModel.build_random(cfg, seed=4)
    g = torch.Generator().manual_seed(0)
    seqs = [torch.randint(0, cfg.vocab, (192,), generator=g) for _ in range(3)]
    ix = LearnedIndexer(cfg, heads=2, dim=16, seed=1)
    hist = warmup(model, ix, seqs[1:], steps=60, lr=3e-3, queries_per_seq=6)
    assert sum(hist[-10:]) < 0.85 * sum(hist[:10]), (hist[:3], hist[-3:])
    # the teacher is a distribution over pages; recall of all pages is the whole mass
    q, k = torch.randn(4, 64), torch.randn(40, 2, 64)
    m = page_mass(q, k, 39)
    assert m.shape == (3,) and abs(float(m.sum()) - 1.0) < 1e-5
    full = topk_recall(model, ix, seqs[0], top_k=64)
    assert abs(full - 1.0) < 1e-4
    sd = ix.state_dict()
    ix2 = LearnedIndexer(cfg, heads=2, dim=16, seed=9)
    ix2.load_state_dict(sd)
    assert abs(topk_recall(model, ix2, seqs[0], top_k=3) - topk_recall(model, ix, seqs[0], top_k=3)) < 1e-6


def test_sparse_engine_accepts_a_learned_indexer():
    import torch
    from helpers import make_engine, rand_prompts
    from tilerl_b200.config import tiny_hybrid
    from tilerl_b200.engine import SamplingParams
    from tilerl_b200.sparse import SparseConfig, SparseKV
    from tilerl_b200.sparse_index import LearnedIndexer
    cfg = tiny_hybrid()
    ix = LearnedIndexer(cfg, heads=2, dim=16)
    sp = SparseKV(cfg, SparseConfig(top_k=64, window=2, refresh_ticks=2, min_tokens=32), indexer=ix)
    dense = make_engine(cfg)
    eng = make_engine(cfg, sparse=sp)
    p = rand_prompts(cfg, 1, 80)
    want = dense.generate(p, SamplingParams(max_tokens=6))[0].tokens
    # k covers every page: the learned scorer may order them freely, the result equals dense
    assert eng.generate(p, SamplingParams(max_tokens=6))[0].tokens == want
    assert sp.stats["sparse_ticks"] > 0


def test_prefix_store_serves_sparse_requests_and_a_hit_equals_the_cold_run():
    """Pages never leave the device here, so the prefix store of the dense path is the sparse one too: a
    follower adopts the publisher's blocks and GDN snapshot, and its page selection reads bounds computed
    from those very pages."""
    from tilerl_b200.kv import PrefixStore
    cfg = tiny_hybrid()
    p = rand_prompts(cfg, 1, 90, seed=8)[0]
    sp = SamplingParams(max_tokens=10)
    mk = lambda: SparseKV(cfg, SparseConfig(top_k=2, window=1, refresh_ticks=2, min_tokens=32))   # noqa: E731
    cold_eng = make_engine(cfg, blocks=200, sparse=mk())
    cold = cold_eng.generate([p], sp)[0]
    mgr = mk()
    eng = make_engine(cfg, blocks=200, model=cold_eng.model, sparse=mgr)
    eng.prefix = PrefixStore(eng.kv)
    first = eng.generate([p], sp)[0]
    warm = eng.generate([p], sp)[0]
    assert first.tokens == cold.tokens == warm.tokens
    assert eng.prefix.hits == 1 and warm.cached_tokens >= 80 and mgr.stats["sparse_ticks"] > 0
    s = eng.stats()
    assert s["sparse_ticks"] > 0 and s["sparse"]["sparse_ticks"] == mgr.stats["sparse_ticks"]
    eng.invalidate_weights()
    assert eng.kv.used_blocks == 0
