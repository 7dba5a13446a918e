import math

import torch

from tilerl_b200.ops import ref


def _gdn_inputs(b=2, t=37, h=3, dk=8, dv=8, seed=0):
    g = torch.Generator().manual_seed(seed)
    q = ref.l2norm(torch.randn(b, t, h, dk, generator=g)) / math.sqrt(dk)
    k = ref.l2norm(torch.randn(b, t, h, dk, generator=g))
    v = torch.randn(b, t, h, dv, generator=g)
    gl = -torch.rand(b, t, h, generator=g) * 0.5
    beta = torch.rand(b, t, h, generator=g)
    s0 = torch.randn(b, h, dk, dv, generator=g) * 0.1
    return q, k, v, gl, beta, s0


def test_gdn_chunked_equals_recurrent():
    q, k, v, g, beta, s0 = _gdn_inputs()
    o1, s1 = ref.gdn_recurrent_batched(q, k, v, g, beta, s0)
    for chunk in (4, 16, 64):
        o2, s2 = ref.gdn_chunked(q, k, v, g, beta, s0, chunk=chunk)
        assert torch.allclose(o1, o2, atol=2e-5), chunk
        assert torch.allclose(s1, s2, atol=2e-5), chunk


def test_gdn_hand_backward_equals_autograd():
    q, k, v, g, beta, s0 = _gdn_inputs(b=1, t=9, h=2, dk=4, dv=5)
    leaves = [x.clone().requires_grad_(True) for x in (q, k, v, g, beta, s0)]
    o, s = ref.gdn_recurrent_batched(*leaves)
    go = torch.randn_like(o)
    gs = torch.randn_like(s)
    want = torch.autograd.grad((o * go).sum() + (s * gs).sum(), leaves)
    got = ref.gdn_recurrent_backward(q, k, v, g, beta, s0, go, gs)
    for a, b in zip(want, got):
        assert torch.allclose(a, b, atol=1e-5)


def test_rope_partial_is_rotation_and_leaves_tail():
    x = torch.randn(5, 2, 16)
    pos = torch.tensor([0, 1, 7, 100, 1000])
    y = ref.rope_partial(x, pos, 1e6, 8)
    assert torch.equal(y[..., 8:], x[..., 8:])
    assert torch.allclose(y[..., :8].norm(dim=-1), x[..., :8].norm(dim=-1), atol=1e-5)
    assert torch.allclose(y[0], x[0])


def test_paged_attention_matches_dense():
    torch.manual_seed(0)
    t, hq, hkv, d = 21, 4, 2, 8
    q = torch.randn(t, hq, d); k = torch.randn(t, hkv, d); v = torch.randn(t, hkv, d)
    gate = torch.randn(t, hq, d)
    kc = torch.zeros(8, hkv, 16, d); vc = torch.zeros(8, hkv, 16, d)
    blocks = [5, 2]
    smap = torch.tensor([blocks[p // 16] * 16 + p % 16 for p in range(t)])
    ref.kv_write(kc, vc, k, v, smap)
    table = torch.tensor([blocks + [0]], dtype=torch.int32)
    out = ref.paged_attention(q, gate, kc, vc, table, torch.zeros(t, dtype=torch.int32),
                              torch.arange(t), 1 / math.sqrt(d))
    want = ref.dense_attention(q[None], k[None], v[None], gate[None], 1 / math.sqrt(d))[0]
    assert torch.allclose(out, want, atol=1e-5)


def test_sharded_ce_equals_full():
    torch.manual_seed(0)
    lg = torch.randn(7, 40)
    tg = torch.randint(0, 40, (7,))
    w = torch.rand(7)
    l0, g0 = ref.cross_entropy_grad(lg, tg, w)
    l1, gs = ref.cross_entropy_sharded([lg[:, :16], lg[:, 16:]], tg, w, [0, 16])
    assert torch.allclose(l0, l1, atol=1e-6)
    assert torch.allclose(g0, torch.cat(gs, -1), atol=1e-6)


def test_sampling_greedy_seeded_and_nucleus():
    lg = torch.tensor([0.1, 3.0, 2.9, -1.0])
    assert ref.sample(lg, 0.0, 1.0, 0, 1)[0] == 1
    a = ref.sample(lg, 1.0, 0.9, 0, ref.sample_seed(5, 3))
    b = ref.sample(lg, 1.0, 0.9, 0, ref.sample_seed(5, 3))
    assert a == b
    toks = {ref.sample(lg, 1.0, 0.5, 0, s)[0] for s in range(40)}
    assert toks <= {1, 2}  # nucleus of mass .5 can only hold the two big logits
    tok, lp = ref.sample(lg, 1.0, 1.0, 1, 0)
    assert tok == 1 and abs(lp) < 1e-6  # top-k=1: probability 1 under the restricted dist


def test_select_pages_window_and_topk():
    scores = torch.tensor([0.1, 5.0, 0.2, 4.0, 0.0, 0.0, 0.0, 0.0])
    assert ref.select_pages(scores, 8, top_k=2, window=3) == [1, 3, 5, 6, 7]
    assert ref.select_pages(scores, 2, top_k=4, window=3) == [0, 1]
