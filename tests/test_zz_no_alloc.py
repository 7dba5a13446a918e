"""Allocation-free attention entry point (``trl_attn_paged_static``).

Some users of this library run where device memory may not be allocated during a call:
the host application owns every byte of the GPU, or a cudaMalloc's device-wide
synchronisation is not acceptable in their serving loop.  For them the split-KV attention
is also exported with its scratch in a fixed device array inside the library.  This test
calls that exported C symbol directly (ctypes, raw pointers) and checks it against the
regular entry point, twice in a row because the scratch keeps the previous call's data.
It lives in a file that sorts last so a failure here cannot hide other tests' results.
"""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _problem(seed):
    g = torch.Generator().manual_seed(seed)
    t, n_q, n_kv, d, blocks = 3, 8, 2, 256, 12
    dev = "cuda"
    q = torch.randn(t, n_q, d, generator=g).to(dev, torch.bfloat16)
    qkv = torch.randn(t, n_q * 2 * d + 2 * n_kv * d, generator=g).to(dev, torch.bfloat16)  # gate source
    kc = torch.randn(blocks, n_kv, 16, d, generator=g).to(dev, torch.bfloat16)
    vc = torch.randn(blocks, n_kv, 16, d, generator=g).to(dev, torch.bfloat16)
    table = torch.tensor([[3, 7, 2, 0], [4, 9, 1, 5]], dtype=torch.int32, device=dev)
    seq_ids = torch.tensor([0, 1, 1], dtype=torch.int32, device=dev)
    positions = torch.tensor([37, 50, 51], dtype=torch.int32, device=dev)
    return dict(t=t, n_q=n_q, n_kv=n_kv, d=d, q=q, qkv=qkv, kc=kc, vc=vc, table=table, seq_ids=seq_ids,
                positions=positions)


def test_static_scratch_entry_point_matches_regular_one():
    from tilerl_b200.ops import native
    lib = ctypes.CDLL(native.lib_path())
    P, I, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    fn = lib.trl_attn_paged_static
    fn.argtypes = [P, P, I, P, P, P, I, P, P, P, I, I, I, I, I, F, I, P]
    fn.restype = I
    need = lib.trl_attn_static_scratch_needed
    need.argtypes = [I, I, I, I]
    need.restype = ctypes.c_size_t
    ref = native.lib().trl_attn_paged
    stream = torch.cuda.current_stream().cuda_stream
    for call, splits in enumerate((4, 2)):     # two calls in a row on the shared scratch
        p = _problem(10 + call)
        t, n_q, n_kv, d = p["t"], p["n_q"], p["n_kv"], p["d"]
        assert need(t, n_q, d, splits) == t * n_q * splits * (d + 2) * 4
        scale = 1.0 / math.sqrt(d)
        want = torch.zeros(t, n_q * d, dtype=torch.bfloat16, device="cuda")
        po = torch.empty(t * n_q * splits * d, dtype=torch.float32, device="cuda")
        pm = torch.empty(t * n_q * splits, dtype=torch.float32, device="cuda")
        pl = torch.empty_like(pm)
        rc = ref(p["q"].data_ptr(), p["qkv"].data_ptr(), p["qkv"].stride(0), p["kc"].data_ptr(), p["vc"].data_ptr(),
                 p["table"].data_ptr(), p["table"].stride(0), p["seq_ids"].data_ptr(), p["positions"].data_ptr(),
                 po.data_ptr(), pm.data_ptr(), pl.data_ptr(), want.data_ptr(), t, n_q, n_kv, d, splits, scale, 1, stream)
        assert rc == 0
        got = torch.zeros_like(want)
        rc = fn(p["q"].data_ptr(), p["qkv"].data_ptr(), p["qkv"].stride(0), p["kc"].data_ptr(), p["vc"].data_ptr(),
                p["table"].data_ptr(), p["table"].stride(0), p["seq_ids"].data_ptr(), p["positions"].data_ptr(),
                got.data_ptr(), t, n_q, n_kv, d, splits, scale, 1, stream)
        assert rc == 0
        torch.cuda.synchronize()
        rel = float((got.float() - want.float()).norm() / want.float().norm())
        assert rel < 2e-2, rel
        assert float(want.float().abs().max()) > 0
    # a problem beyond the fixed scratch is refused, nothing is launched
    rc = fn(None, None, 0, None, None, None, 0, None, None, None, 4096, 64, 8, 256, 32, 1.0, 0, stream)
    assert rc != 0
    assert native.read_error()[0] == 0
