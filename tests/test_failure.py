"""Failure detection without any GPU fault: failures are made on the host (a rank that leaves,
a rank that never joins a collective, an exception inside a tick, a corrupted shard) and the
survivors must learn of them through the store, a short timeout or an error status."""
import os
import time
from datetime import timedelta

import pytest
import torch

from world_helpers import free_port


def _hb_rank(rank, world, port, out, mode):
    import torch.distributed as dist
    from tilerl_b200.parallel.health import Heartbeat, PeerLost
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    store = dist.TCPStore("127.0.0.1", port, world, rank == 0, timeout=timedelta(seconds=20))
    dist.init_process_group("gloo", store=store, rank=rank, world_size=world, timeout=timedelta(seconds=20))
    hb = Heartbeat(store, rank, world, interval_s=0.05)
    t = torch.ones(1)
    dist.all_reduce(t)                       # step 0: everyone is here
    if rank == 1:
        if mode == "leave":
            hb.leave()                       # between steps, nothing in flight
        else:
            hb.stop()                        # silent death: the thread just stops beating
        time.sleep(3.0)
        out.put((rank, "gone"))
        return
    t0 = time.monotonic()
    try:
        while time.monotonic() - t0 < 10:
            hb.check(max_age_s=0.6)          # what a training loop does before its next launch
            time.sleep(0.05)
        out.put((rank, "never noticed"))
    except PeerLost as e:
        out.put((rank, f"lost {e.rank} after {time.monotonic() - t0:.2f}"))
    hb.stop()


@pytest.mark.parametrize("mode", ["leave", "silent"])
def test_heartbeat_reports_a_rank_that_left(mode):
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = free_port()
    procs = [ctx.Process(target=_hb_rank, args=(r, 3, port, out, mode)) for r in range(3)]
    for p in procs:
        p.start()
    res = dict(out.get(timeout=60) for _ in range(3))
    for p in procs:
        p.join(timeout=30)
    assert res[1] == "gone"
    for r in (0, 2):
        assert res[r].startswith("lost 1"), res
        assert float(res[r].split()[-1]) < 5.0


def _timeout_rank(rank, world, port, out):
    import torch.distributed as dist
    from tilerl_b200.parallel.health import CollectiveTimeout, guarded
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=timedelta(seconds=2))
    t = torch.ones(4)
    dist.all_reduce(t)
    if rank == 1:
        time.sleep(6)                        # never joins the second collective
        out.put((rank, "skipped"))
        return
    t0 = time.monotonic()
    try:
        guarded("grad all-reduce", dist.all_reduce, t)
        out.put((rank, "no error"))
    except CollectiveTimeout as e:
        out.put((rank, f"timeout {time.monotonic() - t0:.1f} {e}"))


def test_short_process_group_timeout_ends_a_collective_with_an_error():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = free_port()
    procs = [ctx.Process(target=_timeout_rank, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    res = dict(out.get(timeout=60) for _ in range(2))
    for p in procs:
        p.join(timeout=30)
    assert res[0].startswith("timeout") and "grad all-reduce" in res[0], res
    assert float(res[0].split()[1]) < 6.0


def _order_rank(rank, world, port, out):
    import torch.distributed as dist
    from tilerl_b200.parallel.health import order_agrees
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=timedelta(seconds=20))
    same = order_agrees(["a", "b", "c"])
    names = ["a", "b", "c"] if rank == 0 else ["a", "c", "b"]
    out.put((rank, (same, order_agrees(names))))


def test_order_check_turns_a_mismatch_into_a_message():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = free_port()
    procs = [ctx.Process(target=_order_rank, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    res = dict(out.get(timeout=60) for _ in range(2))
    for p in procs:
        p.join(timeout=30)
    assert res[0] == (True, False) and res[1] == (True, False)


def test_exception_in_a_tick_fails_only_the_running_requests():
    from helpers import make_engine, rand_prompts
    from tilerl_b200.config import tiny_hybrid
    from tilerl_b200.engine import SamplingParams
    cfg = tiny_hybrid()
    eng = make_engine(cfg)
    real = eng.model.forward
    calls = {"n": 0}

    def flaky(*a, **k):
        calls["n"] += 1
        if calls["n"] == 3:
            raise RuntimeError("injected: device returned an error")
        return real(*a, **k)

    eng.model.forward = flaky
    eng.run(batching_window_s=0.0)
    try:
        rid = eng.submit(rand_prompts(cfg, 1, 12)[0], SamplingParams(max_tokens=8))
        deadline = time.time() + 30
        res = None
        while res is None and time.time() < deadline:
            res = eng.take(rid)
            time.sleep(0.01)
        assert res is not None and res.error and "injected" in res.error
        # the engine keeps serving: pools were released, a new request completes
        rid2 = eng.submit(rand_prompts(cfg, 1, 12)[0], SamplingParams(max_tokens=4))
        res2 = None
        while res2 is None and time.time() < deadline:
            res2 = eng.take(rid2)
            time.sleep(0.01)
        assert res2 is not None and not res2.error and len(res2.tokens) == 4
        assert eng.stats()["failed"] == 1
        assert eng.liveness()["degraded"] is None and eng.liveness()["last_progress_age_s"] < 5
    finally:
        eng.stop()


def test_corrupted_train_state_is_refused(tmp_path):
    from tilerl_b200.checkpoint import load_train_state, save_train_state
    p = {"w": torch.randn(8, 8)}
    save_train_state(str(tmp_path), 0, params=p, step=3)
    files = [f for f in os.listdir(tmp_path) if f.endswith(".pt")]
    assert files
    path = os.path.join(tmp_path, files[0])
    blob = bytearray(open(path, "rb").read())
    blob[len(blob) // 2] ^= 0xFF
    open(path, "wb").write(bytes(blob))
    with pytest.raises(Exception):
        load_train_state(str(tmp_path), 0, params={"w": torch.zeros(8, 8)})


def test_device_error_word_becomes_an_exception():
    from tilerl_b200.parallel.health import CommTimeout, raise_on_device_error
    raise_on_device_error(lambda: (0, 0, 0, 0))
    with pytest.raises(CommTimeout, match="code=2 a=1"):
        raise_on_device_error(lambda: (2, 1, 0, 7))


def test_card_guard_with_a_fake_nvml():
    from tilerl_b200.parallel.health import card_guard

    class P:
        def __init__(self, pid, mem):
            self.pid, self.usedGpuMemory = pid, mem

    class Fake:
        def __init__(self, procs):
            self.procs = procs

        def nvmlDeviceGetHandleByIndex(self, i):
            return i

        def nvmlDeviceGetComputeRunningProcesses(self, h):
            return self.procs

    card_guard(0, nvml=Fake([P(os.getpid(), 50 << 30)]))            # our own memory does not count
    card_guard(0, nvml=Fake([P(1, 100 << 20)]))                      # a small foreign context is tolerated
    with pytest.raises(RuntimeError, match="in use by other processes"):
        card_guard(0, nvml=Fake([P(1, 40 << 30)]))


def test_engine_reads_the_device_error_word_every_tick_and_fails_the_tick():
    """A bounded device wait that ran out (here: a fake error word on the third tick, as a TP peer
    that never pushed its partial rows would leave) must not turn into tokens: ``step`` raises
    ``CommTimeout``, the running request ends with that error and the engine serves the next one."""
    from helpers import make_engine, rand_prompts
    from tilerl_b200.config import tiny_hybrid
    from tilerl_b200.engine import SamplingParams
    from tilerl_b200.parallel.health import CommTimeout
    cfg = tiny_hybrid()
    eng = make_engine(cfg)
    reads = {"n": 0}

    def fake_read():
        reads["n"] += 1
        return (1, 5, 3, 17) if reads["n"] == 3 else (0, 0, 0, 0)

    eng.ops.read_device_error = fake_read
    try:
        rid = eng.submit(rand_prompts(cfg, 1, 12)[0], SamplingParams(max_tokens=8))
        with pytest.raises(CommTimeout, match="code=1 a=5 b=3 c=17"):
            for _ in range(10):
                eng.step()
        assert reads["n"] == 3                                   # one read per tick
        res = eng.take(rid)
        assert res is not None and res.error and "device wait gave up" in res.error
        assert eng.stats()["device_errors"] == 1 and eng.liveness()["degraded"]
        out = eng.generate([rand_prompts(cfg, 1, 12)[0]], SamplingParams(max_tokens=4))[0]
        assert len(out.tokens) == 4 and not out.error
    finally:
        del eng.ops.read_device_error
