"""Tensor parallelism on real GPUs: TP-2 (and TP-4/8 when present) logits and greedy tokens
against the single-GPU engine, through the fused peer-memory kernels and CUDA-graph ticks."""
import os
import socket

import pytest
import torch

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, out):
    try:
        _worker_body(rank, world, port, out)
    except Exception:  # noqa: BLE001 - a rank that dies must not leave the parent waiting for its timeout
        import traceback
        out.put(dict(error=f"rank {rank}:\n{traceback.format_exc()}"))
        raise


def _worker_body(rank, world, port, out):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    from tilerl_b200.batch import Batch
    from tilerl_b200.config import small_gpu
    from tilerl_b200.engine import SamplingParams
    from tilerl_b200.factory import build_engine, build_model, make_ops
    from tilerl_b200.ops import native
    from tilerl_b200.parallel.symm import SymmComm
    cfg = small_gpu()
    comm = SymmComm.create(dist.group.WORLD, dev, hmax=cfg.hidden, tmax=512)
    ops = make_ops(dev, tp_comm=comm)
    ops.terms_small = ops.terms_large = 4
    ops.gemv_tokens = 8          # same kernel family for 1..8 rows: these tests compare schedules bit for bit
    model = build_model(cfg, dev, seed=0, tp_rank=rank, tp=world, ops=ops)
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(0, cfg.vocab, (40,), generator=g).tolist() for _ in range(2)]
    eng = build_engine(model, ops, slots=4, max_ctx=256, graph=True, prefix=False)
    res = eng.generate(prompts, SamplingParams(max_tokens=10))
    toks = [r.tokens for r in res]
    # sampled request exercises the full-logits gather
    samp = eng.generate([prompts[0]], SamplingParams(max_tokens=4, temperature=1.0, seed=3))[0].tokens
    samp2 = eng.generate([prompts[0]], SamplingParams(max_tokens=4, temperature=1.0, seed=3))[0].tokens
    torch.cuda.synchronize()
    err = native.read_error()
    if rank == 0:
        # single-GPU control on the same device
        ops1 = make_ops(dev)
        ops1.terms_small = ops1.terms_large = 4
        ops1.gemv_tokens = 8
        m1 = build_model(cfg, dev, seed=0, ops=ops1)
        e1 = build_engine(m1, ops1, slots=4, max_ctx=256, graph=True, prefix=False)
        want = [r.tokens for r in e1.generate(prompts, SamplingParams(max_tokens=10))]
        want_s = e1.generate([prompts[0]], SamplingParams(max_tokens=4, temperature=1.0, seed=3))[0].tokens
        out.put(dict(toks=toks, want=want, samp=samp, samp2=samp2, want_s=want_s, err=err,
                     graph=eng.counters["graph_ticks"], vocab=cfg.vocab))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_tp_engine_matches_single_gpu(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    from tilerl_b200.config import small_gpu
    from tilerl_b200.parallel.mesh import check_alignment
    try:
        check_alignment(small_gpu(), world)
    except ValueError as e:
        pytest.skip(f"the small test model does not divide {world} ways: {e}")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, out)) for r in range(world)]
    for p in procs:
        p.start()
    res = out.get(timeout=600)
    if "error" in res:
        for p in procs:
            p.kill()
        pytest.fail(res["error"])
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    assert res["err"][0] == 0, res["err"]
    assert res["graph"] >= 8
    # greedy tokens: identical up to rare near-ties from the different summation order
    agree = sum(a == b for t, w in zip(res["toks"], res["want"]) for a, b in zip(t, w))
    assert agree >= 18, (res["toks"], res["want"])
    assert res["toks"][0][:3] == res["want"][0][:3]
    # sampling: the random-init model's distribution is almost flat, so the token drawn at a
    # fixed seed moves with rounding-level logit differences between TP degrees; what must hold
    # is that a TP engine repeats itself and draws valid ids through the gathered vocab shards
    assert res["samp"] == res["samp2"] and len(res["samp"]) == 4
    assert all(0 <= t < res["vocab"] for t in res["samp"])
