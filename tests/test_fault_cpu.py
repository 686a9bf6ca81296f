"""Failure detection without faulting any device: failures are made on the host (a rank that raises,
stalls or never joins; a corrupted checkpoint) and the other ranks must notice between steps."""
import datetime
import os
import time

import pytest
import torch
import torch.distributed as dist

from dist_utils import free_port, run_ranks


def _leaving_rank_worker(rank, world, out_dir):
    from kolmogorov_moe_architecture_b200.utils.fault import FaultInjector, HeartbeatMonitor
    store = dist.distributed_c10d._get_default_store()
    hb = HeartbeatMonitor(store, rank, world, timeout_s=5.0)
    inj = FaultInjector(rank=1, step=2, kind="raise")
    done = 0
    stopped_because = None
    for step in range(5):
        try:
            inj.maybe_fail(rank, step)
        except RuntimeError:
            hb.mark_leaving()                      # leaves between steps, nothing in flight
            stopped_because = "self"
            break
        gone = hb.wait_all(step)
        if gone:
            stopped_because = gone
            break
        t = torch.ones(1)
        dist.all_reduce(t)                         # only launched when every rank agreed on this step
        assert t.item() == world
        done += 1
    with open(os.path.join(out_dir, f"r{rank}.txt"), "w") as f:
        f.write(f"{done} {stopped_because}")


def test_rank_that_raises_is_noticed_before_the_next_collective(tmp_path):
    run_ranks(_leaving_rank_worker, 3, str(tmp_path), timeout=60)
    res = {r: open(tmp_path / f"r{r}.txt").read().split(" ", 1) for r in range(3)}
    assert res[1] == ["2", "self"]
    for r in (0, 2):
        assert res[r][0] == "2" and res[r][1] == "[1]"       # two full steps, then stopped because rank 1 left


def _stall_worker(rank, world, out_dir):
    from kolmogorov_moe_architecture_b200.utils.fault import FaultInjector, HeartbeatMonitor, StepWatchdog
    store = dist.distributed_c10d._get_default_store()
    hb = HeartbeatMonitor(store, rank, world, timeout_s=0.6)
    tripped = []
    dog = StepWatchdog(0.4, tripped.append, poll_s=0.05).start()
    inj = FaultInjector(rank=0, step=1, kind="stall", stall_s=1.5)
    verdict = "ok"
    for step in range(3):
        inj.maybe_fail(rank, step)
        gone = hb.wait_all(step)
        if gone:
            verdict = f"late{gone}"
            break
        dog.beat()
    dog.stop()
    with open(os.path.join(out_dir, f"s{rank}.txt"), "w") as f:
        f.write(f"{verdict} {bool(tripped)}")
    time.sleep(1.2)      # let the stalled rank finish before the group is torn down


def test_stalled_rank_trips_watchdog_and_times_out_peers(tmp_path):
    run_ranks(_stall_worker, 2, str(tmp_path), timeout=60)
    assert open(tmp_path / "s1.txt").read().startswith("late[0]")      # peer gave up waiting for rank 0
    assert open(tmp_path / "s0.txt").read().endswith("True")            # rank 0's own watchdog fired


def _never_joins(rank, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE="2")
    dist.init_process_group("gloo", rank=rank, world_size=2, timeout=datetime.timedelta(seconds=3))
    if rank == 1:
        time.sleep(6)                # never enters the collective
        q.put((1, "skipped"))
        return
    t0 = time.time()
    try:
        dist.all_reduce(torch.ones(1))
        q.put((0, "completed"))
    except Exception as e:           # the short process-group timeout ends the collective with an error
        q.put((0, f"error after {time.time() - t0:.1f}s: {type(e).__name__}"))


def test_short_group_timeout_ends_a_collective_nobody_joins():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = free_port()
    ps = [ctx.Process(target=_never_joins, args=(r, port, q)) for r in range(2)]
    for p in ps:
        p.start()
    got = dict(q.get(timeout=60) for _ in range(2))
    for p in ps:
        p.join(20)
        if p.is_alive():
            p.terminate()
    assert got[0].startswith("error"), got


def test_corrupted_checkpoint_is_rejected(tmp_path):
    import kolmogorov_moe_architecture_b200 as kmoe
    from kolmogorov_moe_architecture_b200.training import checkpoint as ck
    cfg = kmoe.get_tiny_debug_config(vocab_size=64, max_seq_len=16)
    m = kmoe.MoETransformer(cfg, verbose=False)
    path = str(tmp_path / "c.pt")
    ck._atomic_save({"model_state_dict": m.state_dict()}, path)
    raw = bytearray(open(path, "rb").read())
    raw[len(raw) // 2: len(raw) // 2 + 64] = b"\0" * 64
    open(path, "wb").write(bytes(raw[: len(raw) * 2 // 3]))          # damaged and truncated
    with pytest.raises(Exception):
        ck.load_model_state(m, path)
    assert not os.path.exists(path + ".tmp")                          # writes go through a temp file + rename
