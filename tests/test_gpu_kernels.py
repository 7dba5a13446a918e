"""Per-kernel parity on a B200: each sm_100a kernel against the fp32 torch oracle of
the same op (``tilerl_b200.ops.ref``), at small shapes that hit every tail and at
the 27B's real shapes."""
import math

import pytest
import torch

from tilerl_b200 import formats as F
from tilerl_b200.ops import ref

pytestmark = pytest.mark.gpu

DEV = "cuda"


@pytest.fixture(scope="module")
def ops():
    from tilerl_b200.ops.cuda import CudaOps
    return CudaOps(DEV)


def _q(n, k, seed=0, std=0.02):
    g = torch.Generator().manual_seed(seed)
    w = torch.randn(n, k, generator=g) * std
    return F.quantize_nvfp4(w).to(DEV)


def _rel(a, b):
    return float((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-9))


@pytest.mark.parametrize("m", [1, 2, 3, 4, 7, 8])
@pytest.mark.parametrize("n,k", [(96, 256), (130, 1024), (5120, 6144), (1031, 17408)])
def test_gemv_nvfp4_plain(ops, m, n, k):
    w = _q(n, k, seed=n + k)
    x = (torch.randn(m, k, generator=torch.Generator().manual_seed(m)) * 2).to(DEV, torch.bfloat16)
    y = torch.empty(m, n, dtype=torch.bfloat16, device=DEV)
    ops.gemv_now(x, w, y)
    want = ref.linear(x, w)
    assert _rel(y, want) < 6e-3
    from tilerl_b200.ops import native
    assert native.read_error()[0] == 0


def test_gemv_nvfp4_fused_norm_residual_swiglu_f32(ops):
    n, k, m = 1024, 5120, 3
    w = _q(n, k, seed=5)
    g = torch.Generator().manual_seed(9)
    x = (torch.randn(m, k, generator=g) * 30).to(DEV, torch.bfloat16)   # large activations: range scaling
    nw = (1 + 0.1 * torch.randn(k, generator=g)).to(DEV)
    y = torch.empty(m, n, dtype=torch.bfloat16, device=DEV)
    ops.gemv_now(x, w, y, norm_w=nw, eps=1e-6)
    h = ref.rmsnorm(x, nw, 1e-6).to(torch.bfloat16)
    assert _rel(y, ref.linear(h, w)) < 6e-3
    res = torch.randn(m, n, generator=g).to(DEV, torch.bfloat16)
    out = res.clone()
    ops.gemv_now(x, w, out, residual=out, epi=1)
    assert _rel(out, ref.linear(x, w, res)) < 6e-3
    act = torch.empty(m, n // 2, dtype=torch.bfloat16, device=DEV)
    ops.gemv_now(x, w, act, norm_w=nw, eps=1e-6, epi=2)
    assert _rel(act, ref.swiglu(ref.linear(h, w))) < 1e-2
    yf = torch.empty(m, n, dtype=torch.float32, device=DEV)
    ops.gemv_now(x, w, yf, epi=3)
    assert _rel(yf, ref.linear(x, w)) < 3e-3


@pytest.mark.parametrize("m", [3, 8, 9, 16])
@pytest.mark.parametrize("n,k", [(4104, 5120), (520, 17408), (24, 512), (1030, 6144), (34816, 5120)])
def test_nvfp4_tensor_core_rows_kernel_matches_oracle(ops, m, n, k):
    """3..16 rows against NVFP4 weights on mma.sync (weights streamed once, f16 activations): every
    epilogue against the fp32 oracle, on row counts that end in a half tile or in fewer than 8 rows,
    with activations staged in one phase (k = 5120), in 2 and in 17 phases (k = 17408 at 8 / 16 rows),
    fewer half tiles than CTAs (n = 24), the largest projection of the 27B; run twice for the same
    bits; with the backend's switch on, its dispatch for these row counts lands on the same kernel."""
    from tilerl_b200.ops import native
    w = _q(n, k, seed=n + k + m)
    g = torch.Generator().manual_seed(m * 7 + n)
    x = (torch.randn(m, k, generator=g) * 20).to(DEV, torch.bfloat16)
    nw = (1 + 0.1 * torch.randn(k, generator=g)).to(DEV)
    res = torch.randn(m, n, generator=g).to(DEV, torch.bfloat16)

    def mma(y, *, norm_w=None, residual=None, epi=0):
        rc = ops.lib.trl_gemv_nvfp4_mma(
            x.data_ptr(), x.stride(0), w.wq.data_ptr(), w.scale.data_ptr(), w.tscale.data_ptr(),
            native.ptr(norm_w), 1e-6, native.ptr(residual), residual.stride(0) if residual is not None else 0,
            y.data_ptr(), y.stride(0), m, n, k, epi, native.stream())
        assert rc == 0, rc
        return y

    h = ref.rmsnorm(x, nw, 1e-6).to(torch.bfloat16)
    y = mma(torch.full((m, n), float("nan"), dtype=torch.bfloat16, device=DEV), norm_w=nw)
    y2 = mma(torch.empty(m, n, dtype=torch.bfloat16, device=DEV), norm_w=nw)
    assert torch.equal(y, y2)
    assert _rel(y, ref.linear(h, w)) < 6e-3
    out = mma(res.clone(), residual=res, epi=1)
    assert _rel(out, ref.linear(x, w, res)) < 6e-3
    act = mma(torch.full((m, n // 2), float("nan"), dtype=torch.bfloat16, device=DEV), norm_w=nw, epi=2)
    assert _rel(act, ref.swiglu(ref.linear(h, w))) < 1e-2
    yf = mma(torch.full((m, n), float("nan"), dtype=torch.float32, device=DEV), epi=3)
    assert _rel(yf, ref.linear(x, w)) < 3e-3
    # the backend sends these row counts here
    if m <= ops.mma_tokens and k <= ops.mma_kmax:
        was = ops.gemv_mma
        ops.gemv_mma = True
        try:
            yd = torch.empty(m, n, dtype=torch.bfloat16, device=DEV)
            ops._linear(x, w, yd, norm_w=nw, eps=1e-6)
            torch.cuda.synchronize()
        finally:
            ops.gemv_mma = was
        assert torch.equal(yd, y)
    assert native.read_error()[0] == 0


@pytest.mark.parametrize("m", [1, 2])
@pytest.mark.parametrize("n,k", [(96, 256), (130, 1152), (5120, 6144), (1030, 17408), (5120, 2176), (640, 5120)])
def test_streamed_gemv_matches_oracle_and_register_kernel(ops, m, n, k):
    """The ring-streamed GEMV (stream layout, bulk copies) against the fp32 oracle and against the
    register-streamed kernel on the checkpoint layout, for every epilogue, with ragged last steps
    (k / 32 not a multiple of 32) and row counts that leave warps uneven shares."""
    from tilerl_b200.ops import native
    from tilerl_b200.ops.gemm_tc import stream_layout, w_stream
    w = _q(n, k, seed=n + k)
    # the device pack kernel states the layout that the torch helper states
    assert torch.equal(w_stream(w), stream_layout(w.wq, w.scale, k))
    g = torch.Generator().manual_seed(m + n)
    x = (torch.randn(m, k, generator=g) * 20).to(DEV, torch.bfloat16)
    nw = (1 + 0.1 * torch.randn(k, generator=g)).to(DEV)
    res = torch.randn(m, n, generator=g).to(DEV, torch.bfloat16)

    def run(stream: bool):
        ops.gemv_stream = stream
        outs = []
        y = torch.empty(m, n, dtype=torch.bfloat16, device=DEV)
        ops.gemv_now(x, w, y, norm_w=nw, eps=1e-6)
        outs.append(y)
        out = res.clone()
        ops.gemv_now(x, w, out, residual=out, epi=1)
        outs.append(out)
        act = torch.empty(m, n // 2, dtype=torch.bfloat16, device=DEV)
        ops.gemv_now(x, w, act, norm_w=nw, eps=1e-6, epi=2)
        outs.append(act)
        yf = torch.empty(m, n, dtype=torch.float32, device=DEV)
        ops.gemv_now(x, w, yf, epi=3)
        outs.append(yf)
        torch.cuda.synchronize()
        return outs

    try:
        new, new2, old = run(True), run(True), run(False)
    finally:
        ops.gemv_stream = True
    h = ref.rmsnorm(x, nw, 1e-6).to(torch.bfloat16)
    gu = ref.linear(h, w).float()
    want = [ref.linear(h, w), ref.linear(x, w, res), torch.nn.functional.silu(gu[:, 0::2]) * gu[:, 1::2],
            ref.linear(x, w).float()]
    for a, a2, b, c in zip(new, new2, old, want):
        assert torch.equal(a, a2)                  # fixed summation order: run twice, same bits
        assert _rel(a, c) < 6e-3
        assert _rel(a, b) < 4e-3
    assert native.read_error()[0] == 0


def test_gemv_bf16_lm_head_shape(ops):
    g = torch.Generator().manual_seed(1)
    n, k = 4099, 5120
    w = (torch.randn(n, k, generator=g) * 0.02).to(DEV, torch.bfloat16)
    x = torch.randn(2, k, generator=g).to(DEV, torch.bfloat16)
    nw = torch.ones(k, device=DEV)
    y = torch.empty(2, n, dtype=torch.float32, device=DEV)
    ops.gemv_now(x, w, y, norm_w=nw, eps=1e-6, epi=3)
    want = ref.linear(ref.rmsnorm(x, nw, 1e-6).to(torch.bfloat16), w)
    assert _rel(y, want) < 2e-3
    tok = ops.argmax(y)
    assert tok.tolist() == want.argmax(-1).tolist()


@pytest.mark.parametrize("m", [3, 5, 8, 11, 16])
def test_gemv_bf16_tensor_core_rows_match_oracle_and_the_fma_kernel(ops, m):
    """3..16 rows against bf16 weights take one tensor-core pass (k summed under a fixed permutation):
    compared with the fp32 oracle, with the FMA kernel two rows at a time, for every epilogue, on an
    N that is no multiple of the 16-row warp tile; run twice for the same bits."""
    from tilerl_b200.ops import native
    g = torch.Generator().manual_seed(10 + m)
    n, k = 4099, 5120
    w = (torch.randn(n, k, generator=g) * 0.02).to(DEV, torch.bfloat16)
    x = torch.randn(m, k, generator=g).to(DEV, torch.bfloat16)
    nw = (1.0 + 0.1 * torch.randn(k, generator=g)).to(DEV)
    res = torch.randn(m, n, generator=g).to(DEV, torch.bfloat16)
    h = ref.rmsnorm(x, nw, 1e-6).to(torch.bfloat16)
    # fp32 logits with the norm fused
    y = torch.full((m, n), float("nan"), dtype=torch.float32, device=DEV)
    ops.gemv_now(x, w, y, norm_w=nw, eps=1e-6, epi=3)
    y2 = torch.empty_like(y)
    ops.gemv_now(x, w, y2, norm_w=nw, eps=1e-6, epi=3)
    assert torch.equal(y, y2)
    want = ref.linear(h, w)
    assert _rel(y, want) < 2e-3
    four = torch.empty_like(y)
    for r0 in range(0, m, 2):
        ops.gemv_now(x[r0:r0 + 2], w, four[r0:r0 + 2], norm_w=nw, eps=1e-6, epi=3)
    assert _rel(y, four) < 1e-4
    assert ops.argmax(y).tolist() == want.argmax(-1).tolist()
    # bf16 store without norm, and the residual epilogue
    yb = torch.empty(m, n, dtype=torch.bfloat16, device=DEV)
    ops.gemv_now(x, w, yb)
    assert _rel(yb, ref.linear(x, w)) < 6e-3
    yr = torch.empty(m, n, dtype=torch.bfloat16, device=DEV)
    ops.gemv_now(x, w, yr, residual=res, epi=1)
    assert _rel(yr, ref.linear(x, w, res)) < 6e-3
    assert native.read_error()[0] == 0


def test_spec_accept_kernel_counts_reproduced_drafts_and_selects_the_state_plane(ops):
    """Greedy acceptance of a verify tick on the device against the host walk: full, partial and zero
    acceptance, a chain of one token, a padded sequence (q_len 0: its state slot stays untouched)."""
    from types import SimpleNamespace
    from tilerl_b200.ops import native
    b, w = 5, 4
    chain = torch.tensor([[7, 11, 12, 13], [7, 11, 12, 13], [7, 11, 12, 13], [9, 0, 0, 0], [0, 0, 0, 0]], dtype=torch.int32)
    tok = torch.tensor([[11, 12, 13, 99], [11, 50, 13, 99], [40, 12, 13, 99], [21, 0, 0, 0], [0, 0, 0, 0]], dtype=torch.int32)
    q_len = torch.tensor([4, 4, 4, 1, 0], dtype=torch.int32)
    slots = torch.tensor([3, 1, 4, 2, 0], dtype=torch.int32)
    want = []
    for r in range(b):
        ok = 0
        while ok + 1 < int(q_len[r]) and int(tok[r, ok]) == int(chain[r, ok + 1]):
            ok += 1
        want.append(ok)
    assert want == [3, 1, 0, 0, 0]
    cur = torch.full((6,), 9, dtype=torch.int32, device=DEV)
    pack = torch.full((b * w + b,), -1, dtype=torch.int32, device=DEV)
    batch = SimpleNamespace(n_seqs=b, n_tokens=b * w, token_ids=chain.flatten().to(DEV), q_len=q_len.to(DEV),
                            state_slots=slots.to(DEV))
    ops.spec_accept(tok.flatten().to(DEV), batch, cur, pack)
    torch.cuda.synchronize()
    assert pack[:b * w].cpu().tolist() == tok.flatten().tolist()
    assert pack[b * w:].cpu().tolist() == want
    assert cur.cpu().tolist() == [9, 1, 0, 3, 0, 9]          # slot 0 (the padded row's) and slot 5 untouched
    assert native.read_error()[0] == 0


@pytest.mark.parametrize("n_pages,k", [(1, 4), (37, 8), (700, 128), (2500, 128)])
def test_quest_score_and_topk_kernels_match_the_torch_selection(ops, n_pages, k):
    """Device page selection against the torch statement of it: Quest upper bounds from the K pages
    (no bounds tensor), and the ascending indices of the k largest, on page tables in shuffled order,
    k >= pages, and scores with ties at the k-th value (lowest page indices win)."""
    from tilerl_b200.ops import native
    from tilerl_b200.sparse import SparseKV, quest_scores
    n_q, n_kv, d = 24, 4, 256
    g = torch.Generator().manual_seed(n_pages + k)
    kc = (torch.randn(n_pages + 3, n_kv, 16, d, generator=g)).to(DEV, torch.bfloat16)
    q = torch.randn(n_q, d, generator=g).to(DEV, torch.bfloat16)
    table = (torch.randperm(n_pages, generator=g) + 2).to(DEV, torch.int32)
    sel = ops.quest_select(q, kc, table, k)
    torch.cuda.synchronize()
    want_scores = quest_scores(q, SparseKV.page_bounds(None, kc, table))
    got_scores = ops.ws.get("quest_scores", (n_pages,), torch.float32)
    assert _rel(got_scores, want_scores) < 1e-5
    kk = min(k, n_pages)
    assert sel.shape == (kk,)
    # selection from the kernel's own scores (fp32 sums in another order may swap near-equal neighbours)
    want = torch.sort(torch.topk(got_scores, kk).indices).values
    assert torch.equal(sel, want)
    # ties: scores quantised to a few values; the kept set is every page above the k-th value plus the
    # lowest-index pages at it
    if n_pages > k:
        tied = torch.randint(0, 5, (n_pages,), generator=g).float().to(DEV)
        out = torch.empty(k, dtype=torch.int64, device=DEV)
        native.check(ops.lib.trl_topk_pages(tied.data_ptr(), n_pages, k, out.data_ptr(), native.stream()), "topk")
        torch.cuda.synchronize()
        kth = torch.sort(tied, descending=True).values[k - 1]
        above = torch.nonzero(tied > kth).flatten()
        at = torch.nonzero(tied == kth).flatten()[:k - above.numel()]
        assert torch.equal(out, torch.sort(torch.cat([above, at])).values)
    assert native.read_error()[0] == 0


_BOUNDS_CHILD = r"""
import ctypes, math, sys, torch
from tilerl_b200.ops import native as N
assert N._PATH.endswith("_C_bounds.so"), N._PATH
lib = N.lib()
dev = "cuda"
n_q, n_kv, d, real_blocks, told_blocks = 8, 2, 256, 32, 8
kc = torch.zeros(real_blocks, n_kv, 16, d, dtype=torch.bfloat16, device=dev)
vc = torch.zeros_like(kc)
rows = n_q * 2 * d + 2 * n_kv * d
qkv = (torch.randn(1, rows, device=dev) * 0.5).to(torch.bfloat16)
ones = torch.ones(d, device=dev)
q = torch.zeros(1, n_q, d, dtype=torch.bfloat16, device=dev)
pos = torch.tensor([40], dtype=torch.int32, device=dev)
res = {}
# site 1: the token's KV slot lies in page 20 -- inside the allocation, beyond the 8 pages the call declares
slot = torch.tensor([20 * 16 + 8], dtype=torch.int32, device=dev)
N.check(lib.trl_attn_prep(qkv.data_ptr(), rows, ones.data_ptr(), ones.data_ptr(), pos.data_ptr(), slot.data_ptr(), q.data_ptr(),
                          kc.data_ptr(), vc.data_ptr(), 1, n_q, n_kv, d, 64, 1e6, 1e-6, 1, told_blocks, N.stream()), "prep")
torch.cuda.synchronize()
res["prep"] = list(N.read_error(True))
res["prep_rows_written"] = int((kc.float().abs().sum((1, 2, 3)) > 0).nonzero().flatten().tolist() == [told_blocks - 1])
# site 2: a block-table entry (page 20) beyond the declared pages, in decode attention
table = torch.tensor([[1, 2, 20, 3]], dtype=torch.int32, device=dev)
seq = torch.zeros(1, dtype=torch.int32, device=dev)
po = torch.zeros(n_q * 4 * d, device=dev); pm = torch.zeros(n_q * 4, device=dev); pl = torch.zeros(n_q * 4, device=dev)
out = torch.zeros(1, n_q * d, dtype=torch.bfloat16, device=dev)
N.check(lib.trl_attn_decode_mma(q.data_ptr(), qkv.data_ptr(), rows, kc.data_ptr(), vc.data_ptr(), table.data_ptr(), 4, told_blocks,
                                seq.data_ptr(), pos.data_ptr(), po.data_ptr(), pm.data_ptr(), pl.data_ptr(), out.data_ptr(),
                                1, n_q, n_kv, d, 1, 1, 1.0 / math.sqrt(d), 1, N.stream()), "decode")
torch.cuda.synchronize()
res["decode"] = list(N.read_error(True))
res["finite"] = bool(torch.isfinite(out.float()).all())
# in range: no error word
table_ok = torch.tensor([[1, 2, 5, 3]], dtype=torch.int32, device=dev)
N.check(lib.trl_attn_decode_mma(q.data_ptr(), qkv.data_ptr(), rows, kc.data_ptr(), vc.data_ptr(), table_ok.data_ptr(), 4, told_blocks,
                                seq.data_ptr(), pos.data_ptr(), po.data_ptr(), pm.data_ptr(), pl.data_ptr(), out.data_ptr(),
                                1, n_q, n_kv, d, 1, 1, 1.0 / math.sqrt(d), 1, N.stream()), "decode")
torch.cuda.synchronize()
res["clean"] = list(N.read_error(True))
print("RESULT", res)
"""


def test_checked_build_records_table_indices_out_of_range_and_clamps_them():
    """The -DTRL_DEBUG_BOUNDS build (loaded in a child process): a KV slot and a block-table entry that
    point past the pages the call declares -- but inside the real allocation, so nothing can leave it --
    are recorded as {bounds, site, index, limit} and clamped; indices in range leave the error word clear."""
    import ast
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    lib = os.path.join(root, "tilerl_b200", "_C_bounds.so")
    assert os.path.exists(lib), "build it: python -m tilerl_b200.build --bounds"
    env = dict(os.environ, TRL_BOUNDS_LIB="1", PYTHONPATH=root)
    r = subprocess.run([sys.executable, "-c", _BOUNDS_CHILD], env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    res = ast.literal_eval(next(l for l in r.stdout.splitlines() if l.startswith("RESULT"))[7:])
    assert res["prep"] == [2, 1, 20 * 16 + 8, 8 * 16]                  # TRL_ERR_BOUNDS, site 1, index, limit
    assert res["prep_rows_written"] == 1                               # the row went to the last declared page
    assert res["decode"][:2] == [2, 2] and res["decode"][2:] == [20, 8]
    assert res["finite"] and res["clean"] == [0, 0, 0, 0]


@pytest.mark.parametrize("n_pages,k", [(5, 8), (300, 64), (2100, 128)])
def test_learned_indexer_selection_on_the_device_matches_the_torch_scores(ops, n_pages, k):
    """Page mean keys (one read of every K page), the indexer's projections (library GEMMs), the
    relu-dot score kernel and the radix-select top-k against ``LearnedIndexer.scores``."""
    from tilerl_b200.config import small_gpu
    from tilerl_b200.ops import native
    from tilerl_b200.sparse_index import LearnedIndexer
    import dataclasses
    n_q, n_kv, d = 8, 2, 256
    cfg = dataclasses.replace(small_gpu(), n_q_heads=n_q, n_kv_heads=n_kv)
    ix = LearnedIndexer(cfg, heads=4, dim=128, seed=3, device=DEV)
    g = torch.Generator().manual_seed(n_pages)
    kc = torch.randn(n_pages + 2, n_kv, 16, d, generator=g).to(DEV, torch.bfloat16)
    q = torch.randn(n_q, d, generator=g).to(DEV, torch.bfloat16)
    table = (torch.randperm(n_pages, generator=g) + 1).to(DEV, torch.int32)
    sel = ops.index_select(ix, 0, q, kc, table, k)
    torch.cuda.synchronize()
    want_scores = ix.scores(0, q, kc, table)
    got_scores = ops.ws.get("quest_scores", (n_pages,), torch.float32)
    assert _rel(got_scores, want_scores) < 1e-3                  # tf32 / summation order of the two GEMMs
    kk = min(k, n_pages)
    assert torch.equal(sel, torch.sort(torch.topk(got_scores, kk).indices).values)
    # the pooled rows themselves
    pooled = ops.ws.get("index_pooled", (n_pages, n_kv * d), torch.float32)
    assert _rel(pooled, kc[table.long()].float().mean(2).reshape(n_pages, -1)) < 1e-6
    assert native.read_error()[0] == 0


def test_quant_kernel_bit_exact_and_dequant(ops):
    g = torch.Generator().manual_seed(3)
    for dtype in (torch.float32, torch.bfloat16):
        w = (torch.randn(257, 512, generator=g) * 0.02).to(DEV, dtype)
        want = F.quantize_nvfp4(w.float())
        got = F.NVFP4Tensor(torch.empty_like(want.wq), torch.empty_like(want.scale), torch.zeros(1, device=DEV))
        ops.quantize_nvfp4_(w, got)
        torch.cuda.synchronize()
        assert torch.equal(got.tscale.cpu(), want.tscale.cpu())
        assert torch.equal(got.scale.view(torch.uint8).cpu(), want.scale.view(torch.uint8).cpu())
        assert torch.equal(got.wq.cpu(), want.wq.cpu())
        d = ops.dequantize_nvfp4(got)
        assert torch.allclose(d.float().cpu(), want.dequant().cpu().to(torch.bfloat16).float(), rtol=0, atol=0)


def test_small_ops(ops):
    g = torch.Generator().manual_seed(4)
    x = torch.randn(5, 1024, generator=g).to(DEV, torch.bfloat16)
    w = torch.rand(1024, generator=g).to(DEV)
    assert _rel(ops._rmsnorm(x, w, 1e-6), ref.rmsnorm(x, w, 1e-6)) < 5e-3
    table = torch.randn(100, 1024, generator=g).to(DEV, torch.bfloat16)
    ids = torch.tensor([3, 99, 0], dtype=torch.int32, device=DEV)
    assert torch.equal(ops.embed(table, ids), table[ids.long()])
    gu = torch.randn(4, 512, generator=g).to(DEV, torch.bfloat16)
    act = torch.empty(4, 256, dtype=torch.bfloat16, device=DEV)
    ops.lib.trl_swiglu(gu.data_ptr(), act.data_ptr(), act.numel(), torch.cuda.current_stream().cuda_stream)
    assert _rel(act, ref.swiglu(gu)) < 5e-3


@pytest.mark.parametrize("d,n_q,n_kv,rot", [(256, 6, 1, 64), (256, 24, 4, 64), (64, 4, 2, 64), (128, 8, 2, 32)])
def test_attention_prep_and_paged(ops, d, n_q, n_kv, rot):
    from tilerl_b200.batch import Batch
    from tilerl_b200.config import ModelConfig, ATTN
    cfg = ModelConfig("t", hidden=64, ffn=64, vocab=64, layer_types=(ATTN,), n_q_heads=n_q, n_kv_heads=n_kv,
                      head_dim=d, rotary_dim=rot, rope_theta=1e7)
    g = torch.Generator().manual_seed(d + n_q)
    # two sequences: a decode row with 37 cached tokens, and a 21-token prefill chunk starting at 5
    seqs = [dict(tokens=[1], start=37, blocks=[3, 7, 2], slot=1),
            dict(tokens=list(range(21)), start=5, blocks=[4, 9], slot=2)]
    batch = Batch.build(seqs, DEV)
    t = batch.n_tokens
    qkv = torch.randn(t, cfg.qkv_rows, generator=g).to(DEV, torch.bfloat16)
    qw = (1 + 0.1 * torch.randn(d, generator=g)).to(DEV)
    kw = (1 + 0.1 * torch.randn(d, generator=g)).to(DEV)
    blocks = 12
    kc0 = (torch.randn(blocks, n_kv, 16, d, generator=g)).to(DEV, torch.bfloat16)
    vc0 = (torch.randn(blocks, n_kv, 16, d, generator=g)).to(DEV, torch.bfloat16)

    class Pool:
        def __init__(self, k, v):
            self.k, self.v = k, v

        def layer(self, i):
            return self.k, self.v

    lp = dict(q_norm=qw, k_norm=kw)
    pool_ref = Pool(kc0.float().clone(), vc0.float().clone())
    from tilerl_b200.ops.backend import RefOps
    want = RefOps().attention(qkv, lp, batch, pool_ref, 0, cfg, n_q, n_kv)
    for splits in (1, 4):
        pool = Pool(kc0.clone(), vc0.clone())
        ops.attn_splits = splits
        got = ops.attention(qkv, lp, batch, pool, 0, cfg, n_q, n_kv)
        ops.attn_splits = 0
        assert _rel(got, want) < 2e-2, splits
        assert _rel(pool.k, pool_ref.k) < 1e-2 and torch.equal(pool.v.float(), pool_ref.v.to(torch.bfloat16).float())


@pytest.mark.parametrize("d,nk,nv", [(128, 2, 6), (64, 4, 4), (128, 16, 48)])
def test_gdn_kernel(ops, d, nk, nv):
    from tilerl_b200.batch import Batch
    from tilerl_b200.config import ModelConfig, GDN
    from tilerl_b200.kv import GdnStatePool
    from tilerl_b200.ops.backend import RefOps
    cfg = ModelConfig("t", hidden=64, ffn=64, vocab=64, layer_types=(GDN,), n_q_heads=2, n_kv_heads=1,
                      head_dim=64, rotary_dim=64, rope_theta=1e6, gdn_k_heads=nk, gdn_v_heads=nv,
                      gdn_head_dim=d)
    g = torch.Generator().manual_seed(d + nv)
    lp = dict(conv=(torch.randn(cfg.gdn_conv_dim, 4, generator=g) * 0.3).to(DEV),
              dt_bias=torch.rand(nv, generator=g).to(DEV), a_log=torch.log(1 + 3 * torch.rand(nv, generator=g)).to(DEV),
              gdn_norm=(1 + 0.1 * torch.randn(d, generator=g)).to(DEV))
    pools = [GdnStatePool(cfg, 4, DEV, planes=4, ring_dtype=torch.bfloat16) for _ in range(3)]
    # tick 1: prefill 19 tokens on slot 1, 3 tokens on slot 2; tick 2: decode; tick 3: verify (keep)
    ticks = [
        ([dict(tokens=list(range(19)), start=0, blocks=[1, 2], slot=1), dict(tokens=[1, 2, 3], start=0, blocks=[3], slot=2)], 0),
        ([dict(tokens=[5], start=19, blocks=[1, 2], slot=1), dict(tokens=[6], start=3, blocks=[3], slot=2)], 0),
        ([dict(tokens=[5, 6, 7], start=20, blocks=[1, 2], slot=1, keep=True)], 3),
    ]
    ops.lib.trl_gdn_set_mma(0)       # this test holds the fp32 token-serial kernels to tight state tolerances
    for seqs, keep in ticks:
        batch = Batch.build(seqs, DEV, keep_steps=keep)
        inp = (torch.randn(batch.n_tokens, cfg.gdn_in_rows, generator=g)).to(DEV, torch.bfloat16)
        want = RefOps().gdn(inp, lp, batch, pools[0], 0, cfg, nk, nv)
        got = ops.gdn(inp, lp, batch, pools[1], 0, cfg, nk, nv).clone()
        assert _rel(got, want) < 2e-2
        assert _rel(pools[1].states, pools[0].states) < 1e-3
        assert torch.equal(pools[1].ring, pools[0].ring)
        # the decode tick ran as one launch (state prefetch, prep, step and gated norm in one kernel);
        # the two-launch path (prep kernel, then scan) must give the same numbers from the same pools
        ops.gdn_fused_decode = False
        try:
            got2 = ops.gdn(inp, lp, batch, pools[2], 0, cfg, nk, nv)
        finally:
            ops.gdn_fused_decode = True
        assert _rel(got, got2) < 3e-3                    # another summation order: a bf16 step here and there
        assert torch.allclose(pools[1].states, pools[2].states, rtol=1e-4, atol=1e-6)
        assert torch.equal(pools[1].ring, pools[2].ring)
        if keep:
            for p in pools:
                p.select_step(1, 1)
    ops.lib.trl_gdn_set_mma(-1)


def test_sample_softmax_kernel_distribution_and_logprob():
    """Device sampler: frequencies follow softmax(logits / T), the log-probability is the
    sampled token's, equal seeds give equal tokens."""
    from tilerl_b200.factory import make_ops
    ops = make_ops("cuda")
    g = torch.Generator().manual_seed(4)
    v = 5003
    logits = (torch.randn(3, v, generator=g) * 2.0).cuda()
    temp = 0.8
    n = 4096
    rows = [1] * n
    seeds = list(range(1000, 1000 + n))
    toks, lps = ops.sample_rows(logits, rows, seeds, [temp] * n)
    toks2, _ = ops.sample_rows(logits, rows, seeds, [temp] * n)
    assert toks == toks2
    p = torch.softmax(logits[1].double().cpu() / temp, -1)
    lp_ref = torch.log(p)
    t = torch.tensor(toks)
    assert float((torch.tensor(lps).double() - lp_ref[t]).abs().max()) < 1e-3
    top = torch.topk(p, 5).indices
    for i in top.tolist():
        freq = float((t == i).float().mean())
        assert abs(freq - float(p[i])) < 4 * (float(p[i]) / n) ** 0.5 + 2e-3, (i, freq, float(p[i]))
    # mean log-probability estimates the negative entropy
    ent = -float((p * lp_ref).sum())
    assert abs(-sum(lps) / n - ent) < 0.15


@pytest.mark.parametrize("v,temp,top_k,top_p", [(5003, 0.8, 20, 0.95), (5003, 1.0, 0, 0.8), (248320, 1.0, 20, 0.95),
                                                 (40000, 0.7, 0, 0.9), (3001, 1.3, 50, 1.0)])
def test_sample_nucleus_kernel_matches_the_restricted_distribution(v, temp, top_k, top_p):
    """Top-k / top-p sampler: every drawn token lies in the oracle's kept set, frequencies and
    log-probabilities follow the renormalised restricted distribution, equal seeds repeat."""
    from tilerl_b200.factory import make_ops
    ops = make_ops("cuda")
    g = torch.Generator().manual_seed(v + top_k)
    logits = (torch.randn(2, v, generator=g) * 3.0).cuda()
    n = 4096
    rows, seeds = [1] * n, list(range(77, 77 + n))
    toks, lps = ops.sample_rows(logits, rows, seeds, [temp] * n, [top_k] * n, [top_p] * n)
    toks2, _ = ops.sample_rows(logits, rows, seeds, [temp] * n, [top_k] * n, [top_p] * n)
    assert toks == toks2
    lg = logits[1].double().cpu() / temp
    if top_k:
        kth = torch.topk(lg, top_k).values[-1]
        lg = torch.where(lg < kth, torch.full_like(lg, float("-inf")), lg)
    p = torch.softmax(lg, -1)
    if top_p < 1.0:
        sp, si = torch.sort(p, descending=True)
        cut = (sp.cumsum(0) - sp) >= top_p
        sp = torch.where(cut, torch.zeros_like(sp), sp)
        p = torch.zeros_like(p).scatter_(0, si, sp)
        p = p / p.sum()
    t = torch.tensor(toks)
    assert bool((p[t] > 0).all()), "a token outside the kept set was drawn"
    assert float((torch.tensor(lps).double() - torch.log(p[t])).abs().max()) < 2e-3
    for i in torch.topk(p, 5).indices.tolist():
        freq = float((t == i).float().mean())
        assert abs(freq - float(p[i])) < 4 * (float(p[i]) / n) ** 0.5 + 2e-3, (i, freq, float(p[i]))


def test_sample_rows_mixed_restrictions_in_one_launch():
    """Rows with and without restrictions share one launch; top_k = 1 is the argmax."""
    from tilerl_b200.factory import make_ops
    ops = make_ops("cuda")
    g = torch.Generator().manual_seed(9)
    logits = (torch.randn(4, 7001, generator=g) * 2.0).cuda()
    toks, lps = ops.sample_rows(logits, [0, 1, 2, 3], [5, 6, 7, 8], [1.0, 0.5, 1.0, 2.0], [1, 0, 0, 3], [1.0, 1.0, 1e-6, 1.0])
    am = logits.argmax(-1).tolist()
    assert toks[0] == am[0] and abs(lps[0]) < 1e-5
    assert toks[2] == am[2] and abs(lps[2]) < 1e-5      # a vanishing nucleus keeps the top token only
    assert toks[3] in torch.topk(logits[3], 3).indices.tolist()
    assert 0 <= toks[1] < 7001 and lps[1] < 0


@pytest.mark.parametrize("norm", [False, True])
def test_lora_add_kernel(norm):
    from tilerl_b200.factory import make_ops
    ops = make_ops("cuda")
    g = torch.Generator().manual_seed(2)
    t, k, n, r = 5, 1536, 777, 16
    x = torch.randn(t, k, generator=g).cuda().to(torch.bfloat16)
    a = (torch.randn(r, k, generator=g) * 0.1).cuda()
    b = (torch.randn(n, r, generator=g) * 0.1).cuda()
    nw = (1 + 0.1 * torch.randn(k, generator=g)).cuda()
    y0 = torch.randn(t, n, generator=g).cuda().to(torch.bfloat16)
    y = y0.clone()
    ops._lora_add(y, x, (a, b, 2.0), nw if norm else None, 1e-6)
    xf = x.float()
    if norm:
        xf = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-6) * nw
    want = y0.float() + 2.0 * (xf @ a.t()) @ b.t()
    assert float((y.float() - want).abs().max()) < 0.03 * float(want.abs().max())


def test_bounded_device_wait_returns_a_status_and_leaves_the_context_usable():
    """A peer flag that nothing sets: the all-reduce finish kernel gives up after its (shortened)
    limit, records the error word and returns; the next kernel runs normally."""
    import ctypes

    from tilerl_b200.factory import make_ops
    from tilerl_b200.ops import native as N
    from tilerl_b200.parallel import symm  # registers the comm signatures  # noqa: F401
    ops = make_ops("cuda")
    lib = N.lib()
    N.register("trl_comm_set_wait_ms", [N.I])
    for fn in ("trl_symm_bytes",):
        getattr(lib, fn).restype = ctypes.c_size_t
    hmax = 256
    nbytes = lib.trl_symm_bytes(hmax, 16)
    p = ctypes.c_void_p()
    N.check(lib.trl_symm_alloc(nbytes, ctypes.byref(p)), "alloc")
    try:
        N.check(lib.trl_comm_set_wait_ms(200), "set_wait")
        table = (ctypes.c_void_p * 8)(p.value, p.value, *([None] * 6))   # "world 2", nobody ever pushes
        res = torch.zeros(1, hmax, dtype=torch.bfloat16, device="cuda")
        out = torch.zeros_like(res)
        N.read_error()                                                    # clear
        t0 = __import__("time").time()
        N.check(lib.trl_allreduce_finish(table, 0, 2, hmax, res.data_ptr(), res.stride(0), out.data_ptr(),
                                         out.stride(0), 1, hmax, N.stream()), "finish")
        torch.cuda.synchronize()
        assert __import__("time").time() - t0 < 5.0
        code, a, b, c = N.read_error()
        assert code != 0 and a == 1, (code, a, b, c)                      # wait site 1 = one-shot flags
        from tilerl_b200.parallel.health import CommTimeout, raise_on_device_error
        with pytest.raises(CommTimeout):
            raise_on_device_error(lambda: (code, a, b, c))
        # the context is alive: an ordinary kernel still runs and is correct
        x = torch.randn(4, 512, device="cuda").to(torch.bfloat16)
        w = torch.ones(512, device="cuda")
        y = ops._rmsnorm(x, w, 1e-6)
        torch.cuda.synchronize()
        ref_y = x.float() * torch.rsqrt(x.float().pow(2).mean(-1, keepdim=True) + 1e-6)
        assert float((y.float() - ref_y).abs().max()) < 0.05
        assert N.read_error()[0] == 0
    finally:
        lib.trl_comm_set_wait_ms(2000)
        lib.trl_symm_free(p)


@pytest.mark.parametrize("lens,hist", [((40, 1, 17), (0, 33, 5)), ((64,), (100,)), ((16, 16), (0, 16))])
def test_tiled_prefill_attention_matches_split_kernel_and_oracle(lens, hist):
    """The tiled tensor-core prefill kernel against the per-token split kernel and the fp32
    oracle: ragged sequences, history already in the paged cache, decode rows riding along."""
    import math as _m
    from tilerl_b200.batch import Batch
    from tilerl_b200.config import small_gpu
    from tilerl_b200.factory import make_ops
    from tilerl_b200.kv import PagedKvPool
    from tilerl_b200.ops.backend import RefOps
    cfg = small_gpu()
    ops = make_ops("cuda")
    g = torch.Generator().manual_seed(7)
    n_q, n_kv, d = cfg.n_q_heads, cfg.n_kv_heads, cfg.head_dim
    rows = n_q * 2 * d + 2 * n_kv * d
    lp = {"q_norm": torch.ones(d, device="cuda"), "k_norm": torch.ones(d, device="cuda")}
    outs = {}
    for mode in ("tiled", "split", "ref"):
        pool = PagedKvPool(cfg, 64, "cuda", dtype=torch.bfloat16 if mode != "ref" else torch.float32)
        o = RefOps() if mode == "ref" else ops
        if mode != "ref":
            ops.prefill_attn = mode == "tiled"
        blk = 1
        seqs_hist, seqs_now = [], []
        for i, (n, h) in enumerate(zip(lens, hist)):
            nb = (n + h + 15) // 16
            blocks = list(range(blk, blk + nb))
            blk += nb
            if h:
                seqs_hist.append(dict(tokens=[0] * h, start=0, blocks=blocks, slot=i + 1))
            seqs_now.append(dict(tokens=[0] * n, start=h, blocks=blocks, slot=i + 1))
        gg = torch.Generator().manual_seed(11)
        for seqs in ([seqs_hist] if seqs_hist else []) + [seqs_now]:
            batch = Batch.build(seqs, "cuda")
            t = sum(len(s_["tokens"]) for s_ in seqs)
            qkv = (torch.randn(t, rows, generator=gg) * 0.5).cuda().to(torch.bfloat16)
            res = o.attention(qkv, lp, batch, pool, 0, cfg, n_q, n_kv)
        outs[mode] = res.float().clone()
    ops.prefill_attn = True
    ref_o = outs["ref"]
    for mode in ("tiled", "split"):
        err = float((outs[mode] - ref_o).abs().max())
        assert err < 0.03 * float(ref_o.abs().max()) + 0.02, (mode, err)
    assert float((outs["tiled"] - outs["split"]).abs().max()) < 0.03


@pytest.mark.parametrize("lens,hist", [((5, 1, 33), (0, 40, 7)), ((1, 1), (200, 17))])
def test_fp8_kv_attention_matches_the_fp8_oracle(lens, hist):
    """e4m3 KV pool on the device: the quantising prep kernel writes the bytes and scales the
    oracle writes (up to a rounding flip of the pre-quantisation value), and attention over the
    fp8 pool matches the oracle over its dequantised pool; both stay close to the bf16 pool."""
    from tilerl_b200.batch import Batch
    from tilerl_b200.config import small_gpu
    from tilerl_b200.factory import make_ops
    from tilerl_b200.kv import PagedKvPool
    from tilerl_b200.ops.backend import RefOps
    cfg = small_gpu()
    ops = make_ops("cuda")
    n_q, n_kv, d = cfg.n_q_heads, cfg.n_kv_heads, cfg.head_dim
    rows = n_q * 2 * d + 2 * n_kv * d
    g = torch.Generator().manual_seed(3)
    lp = {"q_norm": (1.0 + 0.1 * torch.randn(d, generator=g)).cuda(), "k_norm": (1.0 + 0.1 * torch.randn(d, generator=g)).cuda()}
    outs, pools = {}, {}
    for mode in ("cuda_fp8", "cuda_fp8_split", "ref_fp8", "cuda_bf16"):
        fp8 = mode != "cuda_bf16"
        pool = PagedKvPool(cfg, 64, "cuda", dtype=torch.float32 if mode == "ref_fp8" else torch.bfloat16, fp8=fp8)
        o = RefOps() if mode == "ref_fp8" else ops
        ops.prefill_attn = mode != "cuda_fp8_split"     # tiled kernel for chunks of >= 16 tokens, or split-KV only
        blk = 1
        seqs_hist, seqs_now = [], []
        for i, (n, h) in enumerate(zip(lens, hist)):
            nb = (n + h + 15) // 16
            blocks = list(range(blk, blk + nb))
            blk += nb
            if h:
                seqs_hist.append(dict(tokens=[0] * h, start=0, blocks=blocks, slot=i + 1))
            seqs_now.append(dict(tokens=[0] * n, start=h, blocks=blocks, slot=i + 1))
        gg = torch.Generator().manual_seed(11)
        for seqs in ([seqs_hist] if seqs_hist else []) + [seqs_now]:
            batch = Batch.build(seqs, "cuda")
            t = sum(len(s_["tokens"]) for s_ in seqs)
            qkv = (torch.randn(t, rows, generator=gg) * 0.5).cuda().to(torch.bfloat16)
            res = o.attention(qkv, lp, batch, pool, 0, cfg, n_q, n_kv)
        outs[mode] = res.float().clone()
        pools[mode] = pool
    a, b = pools["cuda_fp8"], pools["ref_fp8"]
    used = slice(1, blk)
    for name in ("k", "v"):
        sa, sb = getattr(a, name + "_scale")[0, used], getattr(b, name + "_scale")[0, used]
        assert float(((sa - sb).abs() / sb.abs().clamp_min(1e-20)).max()) < 2e-2, name
        da = getattr(a, name)[0, used].float() * sa.unsqueeze(-1)
        db = getattr(b, name)[0, used].float() * sb.unsqueeze(-1)
        assert float((da - db).abs().max()) < 0.08 * float(db.abs().max()), name   # one e4m3 step at most
        assert float((da - db).abs().mean()) < 0.01 * float(db.abs().max()), name
    ops.prefill_attn = True
    ref_o = outs["ref_fp8"]
    assert float((outs["cuda_fp8"] - ref_o).abs().max()) < 0.03 * float(ref_o.abs().max()) + 0.02
    assert float((outs["cuda_fp8_split"] - ref_o).abs().max()) < 0.03 * float(ref_o.abs().max()) + 0.02
    assert float((outs["cuda_fp8"] - outs["cuda_fp8_split"]).abs().max()) < 0.03
    assert float((outs["cuda_fp8"] - outs["cuda_bf16"]).abs().max()) < 0.08 * float(ref_o.abs().max()) + 0.03
    assert a.k.element_size() == 1


def test_fp8_kv_engine_greedy_tokens_close_to_bf16_pool():
    """The engine serves from an fp8 KV pool on the device: same first greedy tokens as the bf16
    pool on the small model, with the graph decode path on."""
    from tilerl_b200.config import small_gpu
    from tilerl_b200.engine import SamplingParams
    from tilerl_b200.factory import build_engine, build_model, make_ops
    cfg = small_gpu()
    ops = make_ops("cuda")
    model = build_model(cfg, "cuda", seed=1, ops=ops)
    prompt = list(range(5, 45))
    outs = []
    for fp8 in (False, True):
        eng = build_engine(model, ops, device="cuda", slots=2, max_ctx=256, prefix=False, graph=True, kv_fp8=fp8)
        outs.append(eng.generate([prompt], SamplingParams(max_tokens=12, temperature=0.0))[0].tokens)
    same = 0
    for x, y in zip(outs[0], outs[1]):
        if x != y:
            break
        same += 1
    assert same >= 4, (outs, same)


def test_standalone_narrow_decode_binary():
    """csrc/tests/narrow_decode.cu: every e2m1 byte and every e4m3 byte decodes to the value the
    format defines (the binary is built by ``python -m tilerl_b200.build --tests``)."""
    import os
    import subprocess
    from tilerl_b200 import build as b
    exe = os.path.join(b.ROOT, "build", "bin", "narrow_decode")
    if not os.path.exists(exe):
        b.build_tests()
    r = subprocess.run([exe], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0 and "ok" in r.stdout, (r.returncode, r.stdout, r.stderr)


def test_nan_logits_and_wild_token_ids_stay_in_bounds():
    """A row of NaN logits yields token 0 from the argmax (never the internal sentinel, which
    the captured decode tick would feed to the next embedding gather), and an embedding gather
    of an id outside the table writes a zero row and records a bounds error instead of reading."""
    from tilerl_b200.factory import make_ops
    from tilerl_b200.ops import native
    ops = make_ops("cuda")
    native.read_error()
    logits = torch.randn(3, 5000, device="cuda")
    logits[1] = float("nan")
    got = ops.argmax(logits).tolist()
    assert got[1] == 0 and got[0] == int(logits[0].argmax()) and got[2] == int(logits[2].argmax())
    table = torch.randn(100, 256, device="cuda").to(torch.bfloat16)
    ids = torch.tensor([5, 0x7FFFFFFF, -3, 99], dtype=torch.int32, device="cuda")
    x = ops.embed(table, ids).clone()
    torch.cuda.synchronize()
    assert torch.equal(x[0], table[5]) and torch.equal(x[3], table[99])
    assert float(x[1].abs().max()) == 0.0 and float(x[2].abs().max()) == 0.0
    code, a, _, _ = native.read_error()
    assert code == 2 and a == 1          # bounds error raised by the embedding gather
    assert native.read_error()[0] == 0   # reading clears it


@pytest.mark.parametrize("d,nk,nv", [(128, 2, 4), (64, 2, 2)])
def test_gdn_chunk_parallel_scan_matches_serial_scan_and_oracle(d, nk, nv):
    """The chunk-parallel prefill scan against the token-by-token scan kernel (same inputs, same
    start states; fp32 reassociation only) and against the fp32 oracle: ragged prompt lengths, a
    second prefill tick that continues from non-zero states, full and partial chunks."""
    from tilerl_b200.batch import Batch
    from tilerl_b200.config import ModelConfig, GDN
    from tilerl_b200.factory import make_ops
    from tilerl_b200.kv import GdnStatePool
    from tilerl_b200.ops.backend import RefOps
    ops = make_ops("cuda")
    cfg = ModelConfig("t", hidden=64, ffn=64, vocab=64, layer_types=(GDN,), n_q_heads=2, n_kv_heads=1,
                      head_dim=64, rotary_dim=64, rope_theta=1e6, gdn_k_heads=nk, gdn_v_heads=nv,
                      gdn_head_dim=d)
    g = torch.Generator().manual_seed(d + nv)
    lp = dict(conv=(torch.randn(cfg.gdn_conv_dim, 4, generator=g) * 0.3).to(DEV),
              dt_bias=torch.rand(nv, generator=g).to(DEV), a_log=torch.log(1 + 3 * torch.rand(nv, generator=g)).to(DEV),
              gdn_norm=(1 + 0.1 * torch.randn(d, generator=g)).to(DEV))
    lens1, lens2 = (70, 16, 5, 33), (48, 7, 20, 64)
    pools = {k: GdnStatePool(cfg, 6, DEV, planes=1, ring_dtype=torch.bfloat16) for k in ("wy", "serial", "ref")}
    ops.lib.trl_gdn_set_mma(0)
    try:
        for tick, lens in enumerate((lens1, lens2)):
            starts = (0, 0, 0, 0) if tick == 0 else lens1
            seqs = [dict(tokens=[0] * n, start=s, blocks=list(range(1 + 16 * i, 17 + 16 * i)), slot=i + 1)
                    for i, (n, s) in enumerate(zip(lens, starts))]
            batch = Batch.build(seqs, DEV)
            inp = torch.randn(batch.n_tokens, cfg.gdn_in_rows, generator=g).to(DEV, torch.bfloat16)
            want = RefOps().gdn(inp, lp, batch, pools["ref"], 0, cfg, nk, nv).float()
            ops.lib.trl_gdn_set_wy(0)
            serial = ops.gdn(inp, lp, batch, pools["serial"], 0, cfg, nk, nv).float().clone()
            ops.lib.trl_gdn_set_wy(1)
            got = ops.gdn(inp, lp, batch, pools["wy"], 0, cfg, nk, nv).float().clone()
            assert _rel(got, want) < 2e-2
            assert _rel(got, serial) < 2e-3                      # bf16 outputs: at most a rounding flip
            assert _rel(pools["wy"].states, pools["serial"].states) < 1e-5
            assert _rel(pools["wy"].states, pools["ref"].states) < 1e-3
            assert torch.equal(pools["wy"].ring, pools["serial"].ring)
    finally:
        ops.lib.trl_gdn_set_wy(0)      # the default path
        ops.lib.trl_gdn_set_mma(-1)
    from tilerl_b200.ops import native
    assert native.read_error()[0] == 0


@pytest.mark.parametrize("nk,nv", [(2, 4), (16, 48)])
def test_gdn_tensor_core_chunk_kernel_matches_serial_scan_and_oracle(nk, nv):
    """The mma chunk kernel (16-token chunks, bf16 operands, fp32 state) against the fp32
    token-serial scan and the fp32 oracle: lengths around the chunk size, a long prompt, decode
    rows riding along, a second tick that continues from the states of the first; run twice."""
    from tilerl_b200.batch import Batch
    from tilerl_b200.config import ModelConfig, GDN
    from tilerl_b200.factory import make_ops
    from tilerl_b200.kv import GdnStatePool
    from tilerl_b200.ops import native
    from tilerl_b200.ops.backend import RefOps
    ops = make_ops("cuda")
    d = 128
    cfg = ModelConfig("t", hidden=64, ffn=64, vocab=64, layer_types=(GDN,), n_q_heads=2, n_kv_heads=1,
                      head_dim=64, rotary_dim=64, rope_theta=1e6, gdn_k_heads=nk, gdn_v_heads=nv,
                      gdn_head_dim=d)
    g = torch.Generator().manual_seed(nk + nv)
    lp = dict(conv=(torch.randn(cfg.gdn_conv_dim, 4, generator=g) * 0.3).to(DEV),
              dt_bias=torch.rand(nv, generator=g).to(DEV), a_log=torch.log(1 + 3 * torch.rand(nv, generator=g)).to(DEV),
              gdn_norm=(1 + 0.1 * torch.randn(d, generator=g)).to(DEV))
    lens1, lens2 = (1, 15, 16, 17, 300), (31, 1, 48, 2, 212)
    pools = {k: GdnStatePool(cfg, 8, DEV, planes=1, ring_dtype=torch.bfloat16) for k in ("mma", "mma2", "serial", "ref")}
    try:
        for tick, lens in enumerate((lens1, lens2)):
            starts = (0,) * len(lens) if tick == 0 else lens1
            seqs = [dict(tokens=[0] * n, start=s, blocks=list(range(1 + 32 * i, 33 + 32 * i)), slot=i + 1)
                    for i, (n, s) in enumerate(zip(lens, starts))]
            batch = Batch.build(seqs, DEV)
            inp = torch.randn(batch.n_tokens, cfg.gdn_in_rows, generator=g).to(DEV, torch.bfloat16)
            want = RefOps().gdn(inp, lp, batch, pools["ref"], 0, cfg, nk, nv).float()
            ops.lib.trl_gdn_set_mma(0)
            serial = ops.gdn(inp, lp, batch, pools["serial"], 0, cfg, nk, nv).float().clone()
            ops.lib.trl_gdn_set_mma(1)
            got = ops.gdn(inp, lp, batch, pools["mma"], 0, cfg, nk, nv).float().clone()
            got2 = ops.gdn(inp, lp, batch, pools["mma2"], 0, cfg, nk, nv).float().clone()
            assert torch.equal(got, got2) and torch.equal(pools["mma"].states, pools["mma2"].states)
            assert _rel(got, want) < 2e-2, _rel(got, want)
            assert _rel(got, serial) < 1.5e-2, _rel(got, serial)
            assert _rel(pools["mma"].states, pools["ref"].states) < 1e-2, _rel(pools["mma"].states, pools["ref"].states)
            assert torch.equal(pools["mma"].ring, pools["serial"].ring)
    finally:
        ops.lib.trl_gdn_set_mma(-1)
    assert native.read_error()[0] == 0


@pytest.mark.parametrize("w,hist", [(1, (0, 15, 16, 63, 64, 65, 1000)), (8, (0, 9, 250)), (2, (5, 77)), (3, (31, 100))])
@pytest.mark.parametrize("n_q,n_kv", [(24, 4), (8, 2)])
def test_tensor_core_decode_attention_matches_scalar_kernel_and_oracle(w, hist, n_q, n_kv):
    """The mma split-KV kernel (kv-group x window rows as one tile) on decode rows and verify
    windows: contexts that end inside a page, inside a 64-key tile and across many tiles, every
    split count, against the scalar split kernel and the fp32 oracle; run twice for determinism."""
    import dataclasses
    from tilerl_b200.batch import Batch
    from tilerl_b200.config import small_gpu
    from tilerl_b200.factory import make_ops
    from tilerl_b200.kv import PagedKvPool
    from tilerl_b200.ops.backend import RefOps
    cfg = dataclasses.replace(small_gpu(), n_q_heads=n_q, n_kv_heads=n_kv)
    ops = make_ops("cuda")
    assert ops.attn_mma
    d = cfg.head_dim
    rows = n_q * 2 * d + 2 * n_kv * d
    lp = {"q_norm": torch.ones(d, device="cuda"), "k_norm": torch.ones(d, device="cuda")}
    outs = {}
    for mode in ("mma1", "mma4", "mma7", "mma_auto", "mma_auto2", "scalar", "ref"):
        pool = PagedKvPool(cfg, 96, "cuda", dtype=torch.bfloat16 if mode != "ref" else torch.float32)
        o = RefOps() if mode == "ref" else ops
        ops.attn_mma = mode.startswith("mma")
        ops.attn_splits = {"mma1": 1, "mma4": 4, "mma7": 7}.get(mode, 0)
        blk = 1
        seqs_hist, seqs_now = [], []
        for i, h in enumerate(hist):
            nb = (w + h + 15) // 16
            blocks = list(range(blk, blk + nb))
            blk += nb
            if h:
                seqs_hist.append(dict(tokens=[0] * h, start=0, blocks=blocks, slot=i + 1))
            seqs_now.append(dict(tokens=[0] * w, start=h, blocks=blocks, slot=i + 1))
        gg = torch.Generator().manual_seed(13)
        for seqs in ([seqs_hist] if seqs_hist else []) + [seqs_now]:
            batch = Batch.build(seqs, "cuda")
            t = sum(len(s_["tokens"]) for s_ in seqs)
            qkv = (torch.randn(t, rows, generator=gg) * 0.5).cuda().to(torch.bfloat16)
            res = o.attention(qkv, lp, batch, pool, 0, cfg, n_q, n_kv)
        outs[mode] = res.float().clone()
    ops.attn_mma, ops.attn_splits = True, 0
    ref_o = outs["ref"]
    for mode in ("mma1", "mma4", "mma7", "scalar"):
        err = float((outs[mode] - ref_o).abs().max())
        assert err < 0.03 * float(ref_o.abs().max()) + 0.02, (mode, err)
    assert torch.equal(outs["mma_auto"], outs["mma_auto2"])
    for mode in ("mma1", "mma4", "mma7", "mma_auto"):
        assert float((outs[mode] - outs["scalar"]).abs().max()) < 0.03, mode


@pytest.mark.parametrize("n_q,n_kv", [(24, 4), (8, 2)])
def test_fused_decode_attention_layer_equals_the_three_launches(n_q, n_kv):
    """The one-launch form of a decode tick's attention layer (prep + split-KV attention + merge; an
    option of the backend): against the three-launch form
    (outputs, and the K / V rows both write into the pool) and the fp32 oracle, with non-trivial norm
    weights, contexts of 1 key, inside a page, inside a tile and over many tiles, split counts 1, 5 and
    the backend's choice; twice for the same bits; the arrival counters are back at zero."""
    import dataclasses
    from tilerl_b200.batch import Batch
    from tilerl_b200.config import small_gpu
    from tilerl_b200.factory import make_ops
    from tilerl_b200.kv import PagedKvPool
    from tilerl_b200.ops.backend import RefOps
    cfg = dataclasses.replace(small_gpu(), n_q_heads=n_q, n_kv_heads=n_kv)
    assert cfg.head_dim == 256 and cfg.rotary_dim == 64
    ops = make_ops("cuda")
    assert ops.attn_mma and hasattr(ops.lib, "trl_attn_decode_fused")
    d = cfg.head_dim
    rows = n_q * 2 * d + 2 * n_kv * d
    g0 = torch.Generator().manual_seed(5)
    lp = {"q_norm": (1 + 0.2 * torch.randn(d, generator=g0)).cuda(), "k_norm": (1 + 0.2 * torch.randn(d, generator=g0)).cuda()}
    hist = [0, 9, 70, 300, 1000]
    outs, pools = {}, {}
    for mode in ("fused1", "fused5", "fused_auto", "fused_auto2", "three", "ref"):
        pool = PagedKvPool(cfg, 128, "cuda", dtype=torch.bfloat16 if mode != "ref" else torch.float32)
        o = RefOps() if mode == "ref" else ops
        ops.attn_fused = mode.startswith("fused")
        ops.attn_splits = {"fused1": 1, "fused5": 5}.get(mode, 0)
        blk, seqs_hist, seqs_now = 1, [], []
        for i, h in enumerate(hist):
            nb = (1 + h + 15) // 16
            blocks = list(range(blk, blk + nb))
            blk += nb
            if h:
                seqs_hist.append(dict(tokens=[0] * h, start=0, blocks=blocks, slot=i + 1))
            seqs_now.append(dict(tokens=[0], start=h, blocks=blocks, slot=i + 1))
        gg = torch.Generator().manual_seed(13)
        for seqs in (seqs_hist, seqs_now):
            batch = Batch.build(seqs, "cuda")
            t = sum(len(s_["tokens"]) for s_ in seqs)
            qkv = (torch.randn(t, rows, generator=gg) * 0.5).cuda().to(torch.bfloat16)
            res = o.attention(qkv, lp, batch, pool, 0, cfg, n_q, n_kv)
        outs[mode] = res.float().clone()
        kc, vc = pool.layer(0)
        pools[mode] = (kc.float().clone(), vc.float().clone())
    ops.attn_fused, ops.attn_splits = False, 0
    torch.cuda.synchronize()
    ref_o = outs["ref"]
    for mode in ("fused1", "fused5", "fused_auto", "three"):
        err = float((outs[mode] - ref_o).abs().max())
        assert err < 0.03 * float(ref_o.abs().max()) + 0.02, (mode, err)
        assert float((outs[mode] - outs["three"]).abs().max()) < 0.03, mode
        # the pool rows the tick wrote: bf16 roundings of the same fp32 values (the two forms sum the
        # squares of a row in a different order)
        for a, b in zip(pools[mode], pools["three"]):
            assert float((a - b).abs().max()) <= 0.02 * float(b.abs().max()), mode
    assert torch.equal(outs["fused_auto"], outs["fused_auto2"])
    assert int(ops._attn_counters.abs().sum()) == 0
    from tilerl_b200.ops import native
    assert native.read_error()[0] == 0


@pytest.mark.parametrize("m", [1, 2])
@pytest.mark.parametrize("h,ffn,inner", [(1024, 3072, 2048), (5120, 2176, 1152)])
def test_chained_projections_equal_separate_launches(ops, m, h, ffn, inner):
    """A layer's worth of dependent decode projections (norm + in-projection, output projection +
    residual, norm + gate_up + SwiGLU, down projection + residual) queued into one chained launch
    gives the bits of the four separate launches, twice in a row, and matches the fp32 oracle.
    Shapes with K % 1024 != 0 take the ragged-step path inside the chain."""
    from tilerl_b200.ops import native
    g = torch.Generator().manual_seed(h + ffn + m)
    w_in, w_out = _q(2 * inner, h, seed=1), _q(h, inner, seed=2)
    w_gu, w_down = _q(2 * ffn, h, seed=3), _q(h, ffn, seed=4)
    x0 = torch.randn(m, h, generator=g).to(DEV, torch.bfloat16)
    nw1 = (1 + 0.1 * torch.randn(h, generator=g)).to(DEV)
    nw2 = (1 + 0.1 * torch.randn(h, generator=g)).to(DEV)

    def layer(chain: bool):
        ops.chain = chain
        x = x0.clone()
        y = torch.empty(m, 2 * inner, dtype=torch.bfloat16, device=DEV)
        act = torch.empty(m, ffn, dtype=torch.bfloat16, device=DEV)
        launches = native.launch_count
        ops._gemv(x, w_in, y, norm_w=nw1, eps=1e-6)
        a = y[:, :inner]                               # a strided view feeds the next projection
        ops._gemv(a, w_out, x, residual=x, epi=1)
        ops._gemv(x, w_gu, act, norm_w=nw2, eps=1e-6, epi=2)
        ops._gemv(act, w_down, x, residual=x, epi=1)
        ops.flush()
        torch.cuda.synchronize()
        return x, y, act, native.launch_count - launches

    keep = ops.chain
    try:
        c1, c2, s1 = layer(True), layer(True), layer(False)
    finally:
        ops.chain = keep
    assert c1[3] == 1 and s1[3] == 4
    for a, b, c in zip(c1[:3], c2[:3], s1[:3]):
        assert torch.equal(a, b) and torch.equal(a, c)
    h1 = ref.rmsnorm(x0, nw1, 1e-6).to(torch.bfloat16)
    y = ref.linear(h1, w_in).to(torch.bfloat16)
    x1 = ref.linear(y[:, :inner], w_out, x0).to(torch.bfloat16)
    gu = ref.linear(ref.rmsnorm(x1, nw2, 1e-6).to(torch.bfloat16), w_gu).float()
    act = (torch.nn.functional.silu(gu[:, 0::2]) * gu[:, 1::2]).to(torch.bfloat16)
    x2 = ref.linear(act, w_down, x1)
    assert _rel(c1[0], x2) < 1e-2
    assert native.read_error()[0] == 0
