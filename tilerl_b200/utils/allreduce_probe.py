"""Collective micro-benchmarks across the GPUs of one box (torchrun, one rank per GPU):

* the decode tick's pair "row-parallel down projection pushes its partial rows, the gate_up
  projection that follows sums them inside its own launch", against the same two kernels with no
  communication and against NCCL, with the fraction of the roofline (weight stream at the measured
  HBM read rate, or the pushed words at the measured peer-copy rate, whichever is slower);
* the row-parallel projection + all-reduce alone: NCCL (GEMV kernel then
  ``dist.all_reduce`` then residual add) against the fused path (GEMV whose epilogue pushes fp32
  partials into every peer's slot + ``allreduce_finish``), for the down projection of the 27B
  sharded ``world`` ways;
* prefill-sized all-reduce of a ``[T, 5120]`` bf16 tensor: NCCL against the two-shot peer-memory
  kernel (reduce-scatter by peer loads + all-gather by peer stores, residual add fused);
* ZeRO-3 collectives: all-gather of bf16 parameter shards and reduce-scatter (+ scale, fp32 cast)
  of bf16 gradients: NCCL against the peer-load kernels, with bytes received per rank per second
  against the measured NVLink peer-copy figure (770 GB/s per direction).

Every figure is CUDA-event time of a captured CUDA graph of ``reps`` launches where the path can
be captured (the peer-memory kernels), plain event time of ``reps`` eager launches for NCCL, max
over ranks.  Prints one JSON object on rank 0.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \
        -m tilerl_b200.utils.allreduce_probe

Parity: the reference's ``scripts/nccl_probe.py:18-49`` (NCCL sweep 20 KB - 10 MB only).
"""
from __future__ import annotations

import json
import os

import torch
import torch.distributed as dist

NVLINK_PEER_GBS = 770.0


def _time(fn, reps: int, graph: bool) -> float:
    """Microseconds per call."""
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if graph:
        g = torch.cuda.CUDAGraph()
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            with torch.cuda.graph(g, stream=s):
                for _ in range(reps):
                    fn()
        torch.cuda.synchronize()
        dist.barrier()
        g.replay()
        torch.cuda.synchronize()
        dist.barrier()
        a.record()
        g.replay()
        b.record()
    else:
        a.record()
        for _ in range(reps):
            fn()
        b.record()
    torch.cuda.synchronize()
    t = torch.tensor([a.elapsed_time(b) * 1000.0 / reps], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t)


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dev = torch.device("cuda", torch.cuda.current_device())
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    from tilerl_b200.formats import NVFP4Tensor
    from tilerl_b200.ops import native as N_
    from tilerl_b200.factory import make_ops
    from tilerl_b200.parallel.symm import SymmComm
    from tilerl_b200.parallel.zero3 import P2PComm
    h = 5120
    comm = SymmComm.create(dist.group.WORLD, dev, hmax=h, tmax=2048)
    ops = make_ops(dev, tp_comm=comm)
    out = {"world": world}

    # ---- decode: down projection (K = 17408 / world) + all-reduce + residual -----------------
    k = 17408 // world // 32 * 32
    w = NVFP4Tensor(torch.randint(0, 255, (h, k // 2), dtype=torch.uint8, device=dev),
                    (torch.rand(h, k // 16, device=dev) + 0.5).to(torch.float8_e4m3fn), torch.ones(1, device=dev))
    a = torch.randn(1, k, device=dev).to(torch.bfloat16)
    res = comm.xres[:h].view(1, h)
    res.zero_()
    y = torch.zeros(1, h, dtype=torch.bfloat16, device=dev)

    def nccl_path():
        ops.gemv_now(a, w, y)
        dist.all_reduce(y)
        res.add_(y)

    def fused_path():
        comm.linear_allreduce_residual(ops, a, w, res)

    def gemv_only():
        ops.gemv_now(a, w, y)

    out["decode_down_proj"] = dict(
        gemv_only_us=round(_time(gemv_only, 50, True), 2),
        nccl_us=round(_time(nccl_path, 50, False), 2),
        fused_us=round(_time(fused_path, 50, True), 2), k_local=k)
    out["decode_down_proj"]["allreduce_cost_fused_us"] = round(
        out["decode_down_proj"]["fused_us"] - out["decode_down_proj"]["gemv_only_us"], 2)
    out["decode_down_proj"]["allreduce_cost_nccl_us"] = round(
        out["decode_down_proj"]["nccl_us"] - out["decode_down_proj"]["gemv_only_us"], 2)

    # ---- decode: the tick's pattern = row-parallel projection pushes, the next (column-parallel)
    # projection completes the all-reduce inside its own launch, norm folded in -------------------
    from tilerl_b200.ops.cuda import EPI_SWIGLU
    n_up = 2 * 17408 // world
    w_up = NVFP4Tensor(torch.randint(0, 255, (n_up, h // 2), dtype=torch.uint8, device=dev),
                       (torch.rand(n_up, h // 16, device=dev) + 0.5).to(torch.float8_e4m3fn), torch.ones(1, device=dev))
    nw = torch.ones(h, device=dev)
    act = torch.zeros(1, n_up // 2, dtype=torch.bfloat16, device=dev)

    def pair_fused():
        comm.linear_allreduce_residual(ops, a, w, res)
        ops._linear(res, w_up, act, norm_w=nw, eps=1e-6, epi=EPI_SWIGLU)
        ops.flush()

    def pair_local():      # same two projections without any communication (the floor of the pair)
        ops._gemv(a, w, y, residual=res, epi=1)
        ops._linear(y, w_up, act, norm_w=nw, eps=1e-6, epi=EPI_SWIGLU)
        ops.flush()

    def pair_nccl():
        ops.gemv_now(a, w, y)
        dist.all_reduce(y)
        res.add_(y)
        ops._linear(res, w_up, act, norm_w=nw, eps=1e-6, epi=EPI_SWIGLU)
        ops.flush()

    from tilerl_b200.ops.gemm_tc import w_stream
    w_stream(w), w_stream(w_up)
    wbytes = (h * k + n_up * h) * 9 // 16            # e2m1 + e4m3 scale per 16
    link_bytes = h * 8 * (world - 1)                  # {fp32, epoch} words this rank sends, per direction
    hbm_us = wbytes / 6.85e6                          # weight stream at the measured read rate (6.85 TB/s)
    link_us = link_bytes / (NVLINK_PEER_GBS * 1e3)
    fused_us = _time(pair_fused, 50, True)
    comm.settle()
    out["decode_pair_down_then_gate_up"] = dict(
        fused_us=round(fused_us, 2), local_no_comm_us=round(_time(pair_local, 50, True), 2),
        nccl_us=round(_time(pair_nccl, 50, False), 2), weight_bytes=wbytes, link_bytes_per_direction=link_bytes,
        roofline_us=round(max(hbm_us, link_us), 2), roofline_fraction=round(max(hbm_us, link_us) / fused_us, 3))

    # ---- prefill-sized all-reduce ----------------------------------------------------------------
    rows = []
    for t in (16, 128, 512, 2048):
        part = comm.big[: t * h].view(t, h)
        part.normal_()
        resid = comm.xres[: t * h].view(t, h)
        x = torch.randn(t, h, device=dev).to(torch.bfloat16)

        def nccl_ar():
            dist.all_reduce(x)

        def twoshot():
            N_.check(comm.lib.trl_allreduce_twoshot(comm.table, comm.rank, comm.world, comm.hmax, comm.tmax,
                                                    resid.data_ptr(), resid.stride(0), resid.stride(0), t, h,
                                                    N_.stream()), "twoshot")
        us_n = _time(nccl_ar, 20, False)
        us_p = _time(twoshot, 20, True)
        nbytes = t * h * 2
        # each rank receives (world-1)/world of the tensor in the reduce-scatter and again in the all-gather
        wire = 2 * nbytes * (world - 1) / world
        rows.append(dict(tokens=t, bytes=nbytes, nccl_us=round(us_n, 2), twoshot_us=round(us_p, 2),
                         twoshot_wire_gbs=round(wire / us_p / 1e3, 1),
                         twoshot_frac_of_link=round(wire / us_p / 1e3 / NVLINK_PEER_GBS, 3)))
    out["allreduce_bf16_rows_of_5120"] = rows

    # ---- ZeRO-3 collectives -------------------------------------------------------------------------
    zrows = []
    zc = P2PComm(dist.group.WORLD, dev, cap_bytes=(256 << 20) + 4096)
    for mb in (8, 64, 256):
        n_full = mb * (1 << 20) // 2 // (world * 8) * (world * 8)      # bf16 elements of the full unit
        n_sh = n_full // world
        shard = torch.randn(n_sh, device=dev).to(torch.bfloat16)
        full = torch.empty(n_full, dtype=torch.bfloat16, device=dev)
        grad = torch.randn(n_full, device=dev).to(torch.bfloat16)
        gout = torch.zeros(n_sh, dtype=torch.float32, device=dev)
        tmp = torch.empty(n_sh, dtype=torch.bfloat16, device=dev)
        us_ag_n = _time(lambda: dist.all_gather_into_tensor(full, shard), 10, False)
        us_ag_p = _time(lambda: zc.all_gather(shard, full), 10, False)
        us_rs_n = _time(lambda: dist.reduce_scatter_tensor(tmp, grad), 10, False)
        def rs_p2p():          # the kernel runs on the communicator's stream: wait for it, as the optimizer step does
            zc.reduce_scatter(grad, gout, 1.0 / world, True)
            zc.wait()
        us_rs_p = _time(rs_p2p, 10, False)
        recv = n_full * 2 * (world - 1) / world
        zrows.append(dict(unit_mib=mb, allgather_nccl_us=round(us_ag_n, 1), allgather_p2p_us=round(us_ag_p, 1),
                          allgather_p2p_gbs=round(recv / us_ag_p / 1e3, 1),
                          allgather_p2p_frac_of_link=round(recv / us_ag_p / 1e3 / NVLINK_PEER_GBS, 3),
                          reduce_scatter_nccl_us=round(us_rs_n, 1), reduce_scatter_p2p_us=round(us_rs_p, 1),
                          reduce_scatter_p2p_gbs=round(recv / us_rs_p / 1e3, 1),
                          reduce_scatter_p2p_frac_of_link=round(recv / us_rs_p / 1e3 / NVLINK_PEER_GBS, 3)))
    out["zero3_collectives_bf16"] = zrows
    from tilerl_b200.ops import native
    out["device_error_word"] = list(native.read_error())
    if rank == 0:
        print(json.dumps(out))
    dist.barrier()
    zc.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
