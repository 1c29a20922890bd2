"""Failure detection without a GPU fault: a rank that leaves between steps is
noticed on the host by its peers (heartbeat over the store), whether it reports
why or just disappears; and a step that overruns trips the engine watchdog."""
import os
import socket
import time

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _rank(rank, world, port, mode, q):
    from uniserve_v1_b200.parallel.health import Heartbeat, PeerFailure
    store = dist.TCPStore("127.0.0.1", port, world, rank == 0, timeout=__import__("datetime").timedelta(seconds=30))
    dist.init_process_group("gloo", store=store, rank=rank, world_size=world)
    hb = Heartbeat(store, rank, world, interval_s=0.05, timeout_s=2.0)   # a loaded box may stall a beat
    x = torch.ones(4)
    steps = 0
    try:
        for step in range(200):
            hb.check()                       # between steps, nothing in flight
            if rank == 1 and step == 3:
                if mode == "reports":
                    hb.report_failure("numerical_fault: sampled token out of range")
                    time.sleep(0.2)
                os._exit(7)                  # leaves without joining the next collective
            if rank == 0 and step >= 3:
                time.sleep(0.1)              # the survivor idles between steps
                continue
            dist.all_reduce(x)
            steps += 1
    except PeerFailure as e:
        q.put(("detected", e.rank, e.reason, steps))
        hb.close()
        os._exit(0)
    q.put(("not detected", -1, "", steps))
    os._exit(1)


@pytest.mark.parametrize("mode", ["reports", "silent"])
def test_peer_exit_is_detected_between_steps(mode):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank, args=(r, 2, port, mode, q)) for r in range(2)]
    for p in procs:
        p.start()
    what, rank, reason, steps = q.get(timeout=60)
    for p in procs:
        p.join(timeout=30)
    assert what == "detected" and rank == 1 and steps == 3
    if mode == "reports":
        assert "numerical_fault" in reason
    else:
        assert "no heartbeat" in reason
    assert procs[0].exitcode == 0 and procs[1].exitcode == 7


def test_watchdog_flags_an_overrunning_step():
    from uniserve_v1_b200.engine.engine import Watchdog
    wd = Watchdog(0.2)
    assert wd.overdue() is None
    wd.begin("decode step 1")
    assert wd.overdue() is None
    time.sleep(0.4)
    assert "decode step 1" in wd.overdue()
    wd.end()
    assert wd.overdue() is None
