"""Index arithmetic of the CUDA kernels, restated in Python and checked on the CPU.

Each test states one mapping that a kernel relies on (a k permutation, a swizzle, a work split, a
selection rule) the way the kernel's source states it and checks the property the kernel needs
from it: that a permuted dot product is the dot product, that a swizzle is a bijection without bank
conflicts, that a split covers every unit exactly once.  A wrong mapping here is a wrong result (or
an out-of-range access) on the GPU; these run without one.
"""
import numpy as np
import pytest


# ---- csrc/gemv_mma.cu: weights as the A operand of mma.sync m16n8k16 --------------------------------
def _mma_m16n8k16(a_regs, b_regs):
    """The instruction's fragment layout: lane (g, t) = (lane / 4, lane % 4) holds
    A[g][2t..2t+1], A[g+8][2t..], A[g][2t+8..], A[g+8][2t+8..]; B[2t..2t+1][g], B[2t+8..][g];
    C[g][2t], C[g][2t+1], C[g+8][2t], C[g+8][2t+1]."""
    a, b = np.zeros((16, 16)), np.zeros((16, 8))
    for lane in range(32):
        g, t = lane >> 2, lane & 3
        a0, a1, a2, a3 = a_regs[lane]
        a[g, 2 * t:2 * t + 2], a[g + 8, 2 * t:2 * t + 2] = a0, a1
        a[g, 2 * t + 8:2 * t + 10], a[g + 8, 2 * t + 8:2 * t + 10] = a2, a3
        b0, b1 = b_regs[lane]
        b[2 * t:2 * t + 2, g], b[2 * t + 8:2 * t + 10, g] = b0, b1
    return a @ b


def _stage_permuted(x):
    """Activation rows as the kernel stages them: inside a 512-block, k = 128 t + 32 u + 4 i + 2 h + e
    goes to position (((u * 8 + i) * 2 + h) * 4 + t) * 2 + e."""
    xs = np.zeros_like(x)
    for kk in range(0, 512, 2):
        t, u, i, h = kk >> 7, (kk >> 5) & 3, (kk >> 2) & 7, (kk >> 1) & 1
        pos = (((u * 8 + i) * 2 + h) * 4 + t) << 1
        xs[:, pos:pos + 2] = x[:, kk:kk + 2]
    return xs


def test_nvfp4_rows_kernel_k_permutation_and_fragments_give_the_plain_product():
    rng = np.random.default_rng(0)
    w, x = rng.standard_normal((16, 512)), rng.standard_normal((8, 512))
    xs = _stage_permuted(x)
    assert sorted(xs.flatten().tolist()) == sorted(x.flatten().tolist())         # a permutation, nothing lost
    c = np.zeros((16, 8))
    for u in range(4):               # 16-byte piece of the lane's 64-byte run
        for j in range(4):           # 32-bit word of the piece
            for ii in range(2):      # MMA of the word
                chunk = (u * 8 + j * 2 + ii) * 2
                a_regs, b_regs = [], []
                for lane in range(32):
                    g, t = lane >> 2, lane & 3
                    base = 128 * t + 32 * u + 8 * j           # the word's 8 values of rows 2g and 2g + 1
                    ha = [w[2 * g, base + 2 * q:base + 2 * q + 2] for q in range(4)]
                    hb = [w[2 * g + 1, base + 2 * q:base + 2 * q + 2] for q in range(4)]
                    a_regs.append((ha[2 * ii], hb[2 * ii], ha[2 * ii + 1], hb[2 * ii + 1]))
                    # ldmatrix.x2: matrix 0 = rows (tokens) at chunk, matrix 1 at chunk + 1; lane gets row g, elements 2t, 2t+1
                    b_regs.append((xs[g, chunk * 8 + 2 * t:chunk * 8 + 2 * t + 2],
                                   xs[g, (chunk + 1) * 8 + 2 * t:(chunk + 1) * 8 + 2 * t + 2]))
                c += _mma_m16n8k16(a_regs, b_regs)
    got = np.zeros((16, 8))
    for g in range(8):               # fragment row g is weight row 2g, row g + 8 is weight row 2g + 1 (SwiGLU pairs share a lane)
        got[2 * g], got[2 * g + 1] = c[g], c[g + 8]
    assert np.abs(got - w @ x.T).max() < 1e-12


@pytest.mark.parametrize("n_tiles,units", [(1, 1), (2, 34), (3, 34), (15, 10), (16, 10), (16, 34), (5, 12)])
def test_nvfp4_rows_kernel_work_split_covers_every_unit_once_and_spans_three_tiles_at_most(n_tiles, units):
    warps, tot = 12, n_tiles * units
    seen = np.zeros(tot, dtype=int)
    for w in range(warps):
        ua, ub = tot * w // warps, tot * (w + 1) // warps
        seen[ua:ub] += 1
        if ub > ua:
            assert (ub - 1) // units - ua // units <= 2          # three accumulator slots per warp
            # the reduction finds this warp's partial of tile `tile` in slot tile - ua / units
            for tile in range(ua // units, (ub - 1) // units + 1):
                assert 0 <= tile - ua // units < 3
    assert (seen == 1).all()


def test_nvfp4_rows_kernel_phase_count_keeps_the_activation_rows_in_shared_memory():
    budget = 150 * 1024
    for k, rows, want in ((5120, 8, 1), (5120, 16, 2), (6144, 16, 2), (17408, 8, 2), (17408, 16, 17)):
        units = k // 512
        phases = next(d for d in range(1, units + 1) if units % d == 0 and rows * (k // d + 8) * 2 <= budget)
        assert phases == want and units % phases == 0


# ---- csrc/gemv.cu: bf16 weights, 3..16 rows ---------------------------------------------------------
def test_bf16_rows_kernel_lane_chunks_feed_two_mmas_under_one_permutation():
    rng = np.random.default_rng(1)
    w, x = rng.standard_normal((16, 32)), rng.standard_normal((8, 32))     # one 32-wide k step
    c = np.zeros((16, 8))
    for half in range(2):            # elements 0..3 of every lane's 8-value chunk, then 4..7
        a_regs, b_regs = [], []
        for lane in range(32):
            g, t = lane >> 2, lane & 3
            wa, wb, xv = w[g, 8 * t:8 * t + 8], w[g + 8, 8 * t:8 * t + 8], x[g, 8 * t:8 * t + 8]
            o = 4 * half
            a_regs.append((wa[o:o + 2], wb[o:o + 2], wa[o + 2:o + 4], wb[o + 2:o + 4]))
            b_regs.append((xv[o:o + 2], xv[o + 2:o + 4]))
        c += _mma_m16n8k16(a_regs, b_regs)
    assert np.abs(c - w @ x.T).max() < 1e-12


# ---- csrc/attn.cu: decode attention -----------------------------------------------------------------
def _dm_kv_off(key, c):
    r = key & 15
    return (key >> 4) * 8192 + (c >> 3) * 2048 + r * 128 + (((c & 7) ^ (r & 7)) << 4)


def test_decode_attention_tile_swizzle_is_a_bijection_without_bank_conflicts():
    offs = {_dm_kv_off(key, c) for key in range(64) for c in range(32)}
    assert len(offs) == 64 * 32 and min(offs) == 0 and max(offs) == 64 * 512 - 16 and all(o % 16 == 0 for o in offs)
    # an ldmatrix reads the same 16-byte chunk of 8 consecutive keys: eight different bank groups of 16 bytes
    for k0 in range(0, 64, 8):
        for c in range(32):
            assert len({(_dm_kv_off(k0 + i, c) % 128) // 16 for i in range(8)}) == 8
    # what the copy engine writes: a page arrives as four slabs [16 keys][128 B]; inside a slab byte b of key r
    # lands at r * 128 + (((b / 16) ^ (r & 7)) * 16) + b % 16 (the tensor map's 128-byte swizzle)
    for key in (0, 5, 17, 63):
        for c in (0, 7, 8, 31):
            slab, r = c >> 3, key & 15
            assert _dm_kv_off(key, c) == (key >> 4) * 8192 + slab * 2048 + r * 128 + (((c & 7) ^ (r & 7)) << 4)


@pytest.mark.parametrize("n_splits", [1, 4, 37, 64])
def test_decode_attention_splits_cover_every_key_once_for_every_context(n_splits):
    rng = np.random.default_rng(n_splits)
    for kv_len in [1, 15, 16, 17, 127, 128, 129, 576, 4000] + rng.integers(1, 40000, 20).tolist():
        pages = (kv_len + 15) // 16
        n_eff = max(1, min(n_splits, (kv_len + 127) // 128))
        pps = (pages + n_eff - 1) // n_eff
        seen = np.zeros(kv_len, dtype=int)
        for split in range(n_splits):
            lo, hi = split * pps * 16, min(kv_len, (split + 1) * pps * 16)
            if hi > lo:
                assert split < n_eff and lo % 16 == 0
                seen[lo:hi] += 1
        assert (seen == 1).all()


# ---- csrc/sparse.cu: top-k pages by radix select ----------------------------------------------------
def _key(f):
    u = int(np.float32(f).view(np.uint32))
    return (~u & 0xffffffff) if u & 0x80000000 else (u | 0x80000000)


def _topk_model(scores, k):
    """The kernel's steps: four 8-bit passes from the top find the k-th largest key and how many of its
    equals are kept; then every key above it and the first equals in index order."""
    n = len(scores)
    if k >= n:
        return list(range(n))
    keys = [_key(s) for s in scores]
    prefix, need = 0, k
    for p in range(4):
        shift = 24 - 8 * p
        mask = 0 if p == 0 else (0xffffffff << (shift + 8)) & 0xffffffff
        hist = [0] * 256
        for key in keys:
            if key & mask == prefix:
                hist[(key >> shift) & 255] += 1
        b = 255
        while b > 0 and hist[b] < need:
            need -= hist[b]
            b -= 1
        prefix |= b << shift
    out, eq = [], 0
    for i, key in enumerate(keys):
        if key > prefix:
            out.append(i)
        elif key == prefix:
            if eq < need:
                out.append(i)
            eq += 1
    return out


def test_topk_pages_model_equals_sort_with_ties_broken_by_index():
    rng = np.random.default_rng(3)
    for n, k in ((1, 1), (5, 9), (40, 8), (700, 128), (300, 299)):
        for scores in (rng.standard_normal(n).astype(np.float32), rng.integers(-2, 3, n).astype(np.float32)):
            got = _topk_model(scores, k)
            order = sorted(range(n), key=lambda i: (-scores[i], i))[:min(k, n)]
            assert got == sorted(order)
    assert _key(-0.0) < _key(0.0) < _key(1e-30) and _key(-1.0) < _key(-0.5)      # larger float, larger key


# ---- csrc/misc.cu: greedy acceptance of a verify tick -----------------------------------------------
def test_spec_accept_model_equals_the_engines_host_walk():
    rng = np.random.default_rng(4)
    for _ in range(200):
        w = int(rng.integers(1, 9))
        n = int(rng.integers(1, w + 1))
        chain = rng.integers(0, 4, w)
        tok = np.where(rng.random(w) < 0.7, np.roll(chain, -1), rng.integers(0, 4, w))
        ok = 0                                               # the kernel's loop
        while ok + 1 < n and tok[ok] == chain[ok + 1]:
            ok += 1
        drafts, walk = chain[1:n], 0                         # engine._verify_commit
        for k in range(n):
            if k < len(drafts) and tok[k] == drafts[k]:
                walk += 1
                continue
            break
        assert ok == walk


# ---- csrc/zero.cu: source order of the peer-load all-gather -----------------------------------------
@pytest.mark.parametrize("world", [2, 4, 8])
def test_zero_all_gather_source_rotation_reads_every_shard_once_and_spreads_the_readers(world):
    for cta in range(5):
        for rank in range(world):
            assert sorted((rank + k + cta) % world for k in range(world)) == list(range(world))
        for k in range(world):        # at step k the ranks' CTAs of one index read `world` different sources
            assert len({(rank + k + cta) % world for rank in range(world)}) == world
