"""The sort-free top-k / top-p algorithm of the device sampler, as its host model, against the
sorting oracle: same kept set, a draw inside it, the log-probability of the renormalised
restricted distribution."""
import math

import pytest
import torch

from tilerl_b200.ops import ref


def _oracle_probs(lg, temperature, top_k, top_p):
    lg = lg.double() / temperature
    if top_k and top_k < lg.numel():
        kth = torch.topk(lg, top_k).values[-1]
        lg = torch.where(lg < kth, torch.full_like(lg, float("-inf")), lg)
    p = torch.softmax(lg, -1)
    if top_p < 1.0:
        sp, si = torch.sort(p, descending=True)
        cut = (sp.cumsum(0) - sp) >= top_p
        sp = torch.where(cut, torch.zeros_like(sp), sp)
        p = torch.zeros_like(p).scatter_(0, si, sp)
        p = p / p.sum()
    return p


@pytest.mark.parametrize("v,temperature,top_k,top_p", [(1000, 1.0, 20, 0.95), (5000, 0.7, 0, 0.8), (60000, 1.0, 20, 0.95),
                                                       (60000, 1.0, 0, 0.95), (3000, 1.3, 50, 1.0), (777, 1.0, 1, 1.0),
                                                       (777, 2.0, 0, 1e-6)])
def test_model_keeps_the_oracle_set_and_draws_inside_it(v, temperature, top_k, top_p):
    g = torch.Generator().manual_seed(v + top_k)
    lg = torch.randn(v, generator=g) * 3.0
    p = _oracle_probs(lg, temperature, top_k, top_p)
    for u in (0.0, 0.37, 0.999999):
        kept, tok, lp = ref.sample_nucleus_model(lg.numpy(), temperature, top_k, top_p, u)
        assert torch.equal(kept, p > 0)
        assert bool(kept[tok])
        assert abs(lp - math.log(float(p[tok]))) < 1e-3


def test_model_draws_follow_the_restricted_distribution():
    g = torch.Generator().manual_seed(5)
    lg = torch.randn(300, generator=g) * 2.0
    p = _oracle_probs(lg, 0.9, 12, 0.9)
    n = 4000
    counts = torch.zeros(300)
    for i in range(n):
        _, tok, _ = ref.sample_nucleus_model(lg.numpy(), 0.9, 12, 0.9, (i + 0.5) / n)
        counts[tok] += 1
    assert float((counts / n - p.float()).abs().max()) < 2e-3     # stratified u: the inverse CDF itself
