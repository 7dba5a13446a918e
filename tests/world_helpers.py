"""Spawn CPU ranks over gloo for the distributed gates."""
import os
import socket
import traceback

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _entry(rank, world, port, fn, args, out):
    try:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        torch.set_num_threads(1)
        dist.init_process_group("gloo", rank=rank, world_size=world)
        res = fn(rank, world, *args)
        out.put((rank, "ok", res))
        dist.barrier()
        dist.destroy_process_group()
    except Exception:  # noqa: BLE001
        out.put((rank, "error", traceback.format_exc()))


def run_world(world, fn, *args, timeout=300):
    """Run ``fn(rank, world, *args)`` on ``world`` gloo ranks; returns results by rank."""
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = free_port()
    procs = [ctx.Process(target=_entry, args=(r, world, port, fn, args, out)) for r in range(world)]
    for p in procs:
        p.start()
    results = {}
    for _ in range(world):
        rank, status, res = out.get(timeout=timeout)
        if status != "ok":
            for p in procs:
                p.kill()
            raise AssertionError(f"rank {rank} failed:\n{res}")
        results[rank] = res
    for p in procs:
        p.join(timeout=30)
    return [results[r] for r in range(world)]
